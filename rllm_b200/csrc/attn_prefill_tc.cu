// Prefill attention over the paged bfloat16 cache on the 5th-generation tensor cores (tcgen05),
// head sizes 64 and 128: both products of a tile run as UMMA with their accumulators in TMEM.
// The text below gives the sizes for head size 64 (key tiles of 128); with 128 a key tile has 64
// keys, a row's scores are 64, and Q, K and V are two 128-byte atoms wide (see `Shape`).
//
// A work item is a pair of row tiles, 2 x 128 rows: (query token, query head) pairs of ONE kv head
// (row r of a sequence is token r / G, head kvh*G + r % G, as in the mma.sync kernel). Both tiles
// walk the keys they can see in tiles of 128 and share every K and V tile that is fetched:
//   warps 0..2  fetch the Q rows once and the K and V tiles through the block table into 128-byte
//               swizzled shared memory, three stages. Pages of a power of two from 8 keys up come
//               by TMA, one copy per page (or per 128 keys of a larger page) and cache, issued by
//               warp 0 alone and counted by the stage's mbarrier; any other page size comes by
//               16-byte cp.async, the three warps taking turns tile by tile, one stage each;
//   warp 3      one thread issues the products of both row tiles in turn:  S = Q K^T  (M 128,
//               N 128 keys, K 64) into the row tile's S accumulator, and  PV = P V  (M 128, N 64,
//               K 128 keys) with P read from shared memory and V as it lies in the cache tile (an
//               MN-major operand: the contraction runs over key rows);
//   warps 4..7  the softmax of the first row tile, one thread per row; warps 8..11 of the second.
//               A thread reads its row of S (128 scores) from TMEM, takes the maximum, exp2 and
//               the sum in float and writes P as bf16 in the swizzled layout of an A operand.
//               The row's output stays in TMEM, where PV of tile after tile is added up. The
//               exponentials are taken against a maximum that is moved only when the true one
//               has grown by more than 2^8 since (P then stays below 2^8, which bf16 holds as
//               well as values below 1); when it moves, the thread scales its row of the output
//               in TMEM (tcgen05.ld / st) before the next PV is added.
// The (row tile, K tile) steps are numbered k = 0, 1, ... in the order A0 B0 A1 B1 ...; S of step k
// lands in accumulator k % 3, so while both row tiles are in their softmax the scores of the step
// after are computed already, and a row tile that has written its P goes on at once: the four warp
// schedulers always have a warp with work (two warps each, one of either tile).
// TMEM: three S accumulators and PV of both tiles, 512 columns.
// A key j is visible when j <= position of the row and j > position - window.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:573-618 and :328-388 of the reference (scale,
// softmax with the maximum subtracted, weighted V, head h -> kv head h / G, window); unlike the
// reference's prefill kernel a portion also sees what earlier steps left in the cache.
// Every mbarrier wait is bounded; a wait that runs out records an error word and the CTA leaves
// in an orderly way (TMEM freed).
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>
#include <type_traits>
#include <unordered_map>

using namespace rllm;
using namespace sm100;

namespace {

constexpr int PM = 128;          // rows per row tile
constexpr int RT = 2;            // row tiles per work item
constexpr int LOADERS = 3;       // loader warps
constexpr int MMA_WARP = LOADERS;
constexpr int SOFTMAX_WARP0 = LOADERS + 1;      // a multiple of 4: warp w reads TMEM lanes 32 (w % 4) ...
static_assert(SOFTMAX_WARP0 % 4 == 0, "softmax warp w must own TMEM lane quadrant w % 4");
constexpr int THREADS = (LOADERS + 1 + 4 * RT) * 32;
// registers per thread: 168 each at launch (65,536 / 384, in eights); then 4 warps keep 56 and 8 warps have 224
constexpr int REGS_LOW = 56, REGS_HIGH = 224;
static_assert(SOFTMAX_WARP0 * 32 * REGS_LOW + 4 * RT * 32 * REGS_HIGH <= 168 * THREADS, "more registers than the launch has");
constexpr int KV_TILE_BYTES = 16384;             // one K or V tile: 128 keys of 64 values, or 64 keys of 128
constexpr int KVS = 4;           // K/V stages with TMA (one loader, tile after tile). Without TMA only LOADERS of them
                                 // are used: loader warp w always fills stage w (tiles w, w + 3, ...), so its waits
                                 // on that stage's barriers follow one another phase by phase; a warp that moved
                                 // between stages could be two phases ahead, which a parity cannot tell
constexpr int SB = 3;            // S accumulators: one per row tile in its softmax, one being computed ahead
constexpr int TMEM_COLS = 512;

// Sizes that follow from the head size (64 or 128). Operands lie in shared memory as "atoms" of
// 128-byte rows (64 values), swizzled: a tile wider than 64 values is several atoms one after the other.
template <int HD> struct Shape {
  static_assert(HD == 64 || HD == 128, "head sizes 64 and 128");
  static constexpr int PN = HD == 64 ? 128 : 64;     // keys per tile (a K or V tile is 16 KB either way)
  static constexpr int HA = HD / 64;                 // atoms along the head dimension (Q, K, V)
  static constexpr int KA = PN / 64;                 // atoms along the keys (P)
  static constexpr int ATOM_ROWS = PM * 128;         // bytes of one atom of Q or P (128 rows)
  static constexpr int ATOM_KEYS = PN * 128;         // bytes of one atom of K or V (PN rows)
  static constexpr int Q_BYTES = HA * ATOM_ROWS;     // one row tile of Q
  static constexpr int P_BYTES = KA * ATOM_ROWS;     // one row tile of P
  static constexpr int SMEM_BYTES = 1024 + RT * Q_BYTES + 2 * KVS * KV_TILE_BYTES + RT * P_BYTES;   // Q[2], K[KVS], V[KVS], P[2]
  static constexpr int S_COL = 0, O_COL = SB * PN;   // TMEM: three S accumulators, then the output of both row tiles
  static_assert(O_COL + RT * HD <= TMEM_COLS, "S and the outputs must fit in TMEM");
  static_assert(HA * ATOM_KEYS == KV_TILE_BYTES, "a K or V tile is 16 KB");
};

struct PfParams {
  const bf16* q; int q_stride;
  const bf16* kc; const bf16* vc;
  bf16* out; int out_stride;
  const int* cu_q; const int* kv_lens; const int* block_table; int bt_stride;
  int nh, nkv, page_size, page_shift, window;
  int box_rows;          // TMA variant: keys per copy = min(page size, 128)
  int row_pairs, num_seqs, sm_count;
  float scale_log2e;
  int* err;
};

__device__ __forceinline__ float fast_exp2(float x) {          // exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async16z(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;                         // 0 bytes read: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// instruction descriptor: bf16 x bf16 -> f32, A K-major, B K-major or MN-major
__host__ __device__ constexpr uint32_t idesc(int M, int N, bool b_mn_major) {
  return umma_idesc_bf16(M, N) | (b_mn_major ? (1u << 16) : 0u);
}

// TMA: the K and V tiles come by tensor copies over the caches seen as [pages * kv heads][page size][HD].
template <int HD, bool TMA>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const PfParams p) {
  extern __shared__ uint8_t pf_smem_raw[];
  __shared__ __align__(8) uint64_t kv_full[KVS], kv_empty[KVS], s_full[SB], s_free[SB], p_full[RT], pv_full[RT], q_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)pf_smem_raw + 1023) & ~(uintptr_t)1023);
  typedef Shape<HD> C;
  constexpr int PN = C::PN;
  const uint32_t q_s = smem_u32(smem);
  const uint32_t k_s = q_s + RT * C::Q_BYTES, v_s = k_s + KVS * KV_TILE_BYTES, p_s = v_s + KVS * KV_TILE_BYTES;

  const int G = p.nh / p.nkv;
  constexpr int NST = TMA ? KVS : LOADERS;              // K/V stages in use
  if (threadIdx.x == 0) abort_flag = 0;
  if (TMA) {
    // A copy brings whole pages: rows past a sequence's last key keep what the stage held before.
    // The scores of such keys are masked, and their weights are exact zeros, but zero times what
    // an earlier kernel left here need not be zero: start from zeros (later leftovers are keys).
    if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_k); prefetch_tensormap(&tmap_v); }
    uint4* kv = reinterpret_cast<uint4*>(smem + RT * C::Q_BYTES);
    for (int i = threadIdx.x; i < 2 * KVS * KV_TILE_BYTES / 16; i += THREADS) kv[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&tmem_base_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch();
  pdl_wait();                                           // q and the newest keys come from the kernel before
  const uint32_t tmem_base = tmem_base_slot;

  // The CTAs (one per SM) share the (pair of row tiles, kv head, sequence) items out among
  // themselves: items are numbered from the row tiles that see the most keys down, and round r
  // gives CTA c item r * C + c, or r * C + (C - 1 - c) in odd rounds, so that every CTA gets a
  // like share of long and short ones.
  // The warps 0..3 (loaders, products) need few registers, the softmax warps many (a row of 128
  // scores each): the first warpgroup gives registers up, the other two take them, and each side
  // walks the items in its own copy of the loop (the block-wide barriers are the same ones).
  auto walk = [&](auto softmax_side) {
  constexpr bool SOFTMAX = decltype(softmax_side)::value;
  const int items = p.row_pairs * p.nkv * p.num_seqs;
  for (int round = 0;; ++round) {
  const int item = round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  if (item >= items) break;
  const int tile0 = (p.row_pairs - 1 - item / (p.nkv * p.num_seqs)) * RT;      // first of the item's row tiles
  const int kvh = item % p.nkv, seq = (item / p.nkv) % p.num_seqs;
  // an item beyond its sequence's rows (a short portion beside long ones) is skipped by all threads alike
  if (tile0 * PM >= (p.cu_q[seq + 1] - p.cu_q[seq]) * G) continue;
  __syncthreads();                                      // everybody has left the item before
  if (threadIdx.x == 0) {
    for (int i = 0; i < KVS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < SB; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); }
    for (int i = 0; i < RT; ++i) { mbar_init(&p_full[i], 4); mbar_init(&pv_full[i], 1); }
    mbar_init(&q_full, TMA ? 4 * RT : RT);             // TMA: one arrival per softmax warp, which brings its own rows of Q
    fence_barrier_init();
  }
  __syncthreads();
  if (abort_flag) break;                                // a wait ran out in an earlier item: the kernel's output is void anyway

  const int q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q0;
  const int kv_len = p.kv_lens[seq];
  const int rows_total = q_len * G;
  // keys the item's rows can see at all: from the first row's window (or 0) to the last row's position.
  // The later row tile sees at least as far as the earlier one; both start from the same tile.
  int kv_begin = 0, n_t[RT];
  {
    const int p_min = kv_len - q_len + (tile0 * PM) / G;
    if (p.window > 0 && p_min - p.window + 1 > 0) kv_begin = (p_min - p.window + 1) / PN * PN;
#pragma unroll
    for (int g = 0; g < RT; ++g) {
      const bool active = (tile0 + g) * PM < rows_total;         // uniform: a row tile beyond the sequence's rows is empty
      const int p_max = kv_len - q_len + min(q_len - 1, ((tile0 + g) * PM + PM - 1) / G);
      n_t[g] = active ? (p_max + 1 - kv_begin + PN - 1) / PN : 0;
    }
  }
  const int n_tiles = max(n_t[0], n_t[1]);
  // step k is (row tile, K tile) = (k & 1, k >> 1) while both row tiles have tiles left, then the later one alone
  const int n_both = min(n_t[0], n_t[1]), g_long = n_t[1] > n_t[0] ? 1 : 0, n_steps = n_t[0] + n_t[1];

  // Q rows r0 .. r0 + n - 1 of the item (one warp), rows beyond the sequence zero
  auto load_q = [&](int r0, int n) {
    const int ch = lane & 7, rbase = lane >> 3;
#pragma unroll 4
    for (int i = 0; i < n / 4; ++i) {
      const int r = r0 + rbase + 4 * i;                  // row of the item: row tile r / 128, row r % 128 of it
      const int row = tile0 * PM + r;
      const bool valid = row < rows_total;
      const int tok = valid ? row / G : 0, head = kvh * G + (valid ? row % G : 0);
      const bf16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)head * HD + ch * 8;
      const uint32_t dst = q_s + (uint32_t)((r / PM) * C::Q_BYTES + (r % PM) * 128 + ((ch ^ (r & 7)) << 4));
#pragma unroll
      for (int a = 0; a < C::HA; ++a) cp_async16z(dst + (uint32_t)(a * C::ATOM_ROWS), src + a * 64, valid);
    }
  };

  if constexpr (!SOFTMAX) {
  // ---- the products. Step k is (row tile g, K tile t); its S lands in accumulator k % 3.
  constexpr uint32_t id_s = idesc(PM, PN, false);
  constexpr uint32_t id_pv = idesc(PM, 64, true);       // 64 output values at a time
  auto step = [&](int k, int& g, int& t) {
    if (k < 2 * n_both) { g = k & 1; t = k >> 1; } else { g = g_long; t = n_both + (k - 2 * n_both); }
  };
  // descriptors move with the address: 16 bytes are one unit of the start-address field
  const uint64_t dq0 = umma_desc_sw128(q_s), dk0 = umma_desc_sw128(k_s), dv0 = umma_desc_sw128(v_s),
                 dp0 = umma_desc_sw128(p_s);
  auto issue_s = [&](int k, bool& ok) {                 // S = Q K^T of step k (one thread)
    int g, t;
    step(k, g, t);
    const int ks = t % NST;
    if (k >= SB) {
      // the accumulator's scores of step k - 3 are in their threads' registers
      if (!mbar_wait(&s_free[k % SB], (uint32_t)(k / SB - 1) & 1u, &abort_flag)) {
        abort_flag = 1; record_failure(p.err, 28, k); ok = false; return;
      }
    }
    if (!mbar_wait(&kv_full[ks], (uint32_t)(t / NST) & 1u, &abort_flag)) {
      abort_flag = 1; record_failure(p.err, 22, t); ok = false; return;
    }
    tc_fence_after();
    const uint64_t dq = dq0 + (uint64_t)(g * (C::Q_BYTES >> 4)), dk = dk0 + (uint64_t)(ks * (KV_TILE_BYTES >> 4));
    const uint32_t acc = tmem_base + C::S_COL + (uint32_t)(k % SB) * PN;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)                // 16 values a product: atom kk / 4, 32 bytes on within it
      umma_bf16(acc, dq + (uint64_t)((kk >> 2) * (C::ATOM_ROWS >> 4) + (kk & 3) * 2),
                dk + (uint64_t)((kk >> 2) * (C::ATOM_KEYS >> 4) + (kk & 3) * 2), id_s, kk > 0);
    umma_commit(&s_full[k % SB]);
  };
  auto issue_pv = [&](int k, bool& ok) {                // PV of step k, added to the row tile's output (one thread)
    int g, t;
    step(k, g, t);
    // P of this step is written (and the row tile's PV before is complete: its threads waited for it)
    if (!mbar_wait(&p_full[g], (uint32_t)t & 1u, &abort_flag)) {
      abort_flag = 1; record_failure(p.err, 23, t); ok = false; return;
    }
    tc_fence_after();
    const uint64_t dp = dp0 + (uint64_t)(g * (C::P_BYTES >> 4)), dv = dv0 + (uint64_t)((t % NST) * (KV_TILE_BYTES >> 4));
    const uint32_t acc = tmem_base + C::O_COL + (uint32_t)g * HD;
#pragma unroll
    for (int a = 0; a < C::HA; ++a)                     // 64 output values = one atom of V
#pragma unroll
      for (int ks = 0; ks < PN / 16; ++ks) {
        // P: K-major, atoms of 64 keys, 32 bytes per 16 keys; V: MN-major, 16 key rows = 2 KB per step
        umma_bf16(acc + (uint32_t)(a * 64), dp + (uint64_t)((ks >> 2) * (C::ATOM_ROWS >> 4) + (ks & 3) * 2),
                  dv + (uint64_t)(a * (C::ATOM_KEYS >> 4) + ks * (2048 >> 4)), id_pv, t > 0 || ks > 0);
      }
    umma_commit(&pv_full[g]);
    if (g == 1 || t >= n_both) umma_commit(&kv_empty[t % NST]);     // the last reader of this K and V stage
  };
  if (warp < LOADERS && TMA) {
    // ------------------------------------------------------------ loader (TMA): warp 0 alone, tile after tile.
    // Lane c looks up the page of the tile's c-th copy; lane 0 tells the stage's barrier how many
    // bytes are coming; every lane with a page issues its two copies. Nothing waits for a tile to
    // land: up to NST tiles are on their way.
    if (warp == 0) {
      const int* bt = p.block_table + (size_t)seq * p.bt_stride;
      const int copies = PN / p.box_rows;                  // runs of keys per tile; each is one copy per atom and cache
      const uint32_t copy_bytes = (uint32_t)p.box_rows * 128;
      const int cp = lane / C::HA, at = lane % C::HA;      // this lane's run of keys and its atom of 64 values
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % NST;
        if (t >= NST) {
          int w_ok = 1;
          if (lane == 0 && !mbar_wait(&kv_empty[s], (uint32_t)(t / NST - 1) & 1u, &abort_flag)) {
            abort_flag = 1; record_failure(p.err, 21, t); w_ok = 0;
          }
          if (__shfl_sync(0xffffffffu, w_ok, 0) == 0) break;
        }
        const int j = kv_begin + t * PN + cp * p.box_rows;              // first key of this lane's copy
        const bool mine = cp < copies && j < kv_len;
        const int page = mine ? __ldg(bt + (j >> p.page_shift)) : 0;
        const uint32_t n = __popc(__ballot_sync(0xffffffffu, mine));
        if (lane == 0) mbar_expect_tx(&kv_full[s], 2 * n * copy_bytes);
        __syncwarp();
        if (mine) {
          const uint32_t dst = (uint32_t)s * KV_TILE_BYTES + (uint32_t)at * C::ATOM_KEYS + (uint32_t)cp * copy_bytes;
          const int off = j & (p.page_size - 1);
          tma_load_3d(k_s + dst, &tmap_k, &kv_full[s], at * 64, off, page * p.nkv + kvh);
          tma_load_3d(v_s + dst, &tmap_v, &kv_full[s], at * 64, off, page * p.nkv + kvh);
        }
      }
    } else if (warp == 2) {
      // (Q comes from the softmax warps, each thread its own row: one warp fetching a row tile spent 5 us
      // of every item on the addresses of its 1,024 copies)
      if (lane == 0 && n_steps > 0) {
        // ... and warp 2 then issues the S products, as far ahead as accumulators are free
        bool ok = true;
        if (!mbar_wait(&q_full, 0u, &abort_flag)) { abort_flag = 1; record_failure(p.err, 27, 0); ok = false; }
        for (int k = 0; k < n_steps && ok; ++k) issue_s(k, ok);
      }
    }
  } else if (warp < LOADERS) {
    // ------------------------------------------------------------ loaders (any page size): warp w fetches the
    // tiles w, w + 3, ... whole, waits until they have landed and announces them at once, so a
    // tile is ready long before its turn (up to NST tiles are on the way, from different warps).
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;
    const int ch = lane & 7;                              // this lane's 16-byte chunk of a 128-byte row
    const int rbase = lane >> 3;                          // its rows: rbase + 4 i, i < PN / 4
    for (int t = warp; t < n_tiles; t += LOADERS) {
      const int s = t % NST;
      if (t >= NST) {
        int w_ok = 1;
        if (lane == 0 && !mbar_wait(&kv_empty[s], (uint32_t)(t / NST - 1) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 21, t); w_ok = 0;
        }
        if (__shfl_sync(0xffffffffu, w_ok, 0) == 0) break;
      }
      if (t == 0) load_q(0, RT * PM);                     // lands with the tile, announced by its barrier
      const int j0 = kv_begin + t * PN;
      const uint32_t kd = k_s + (uint32_t)s * KV_TILE_BYTES, vd = v_s + (uint32_t)s * KV_TILE_BYTES;
#pragma unroll 1
      for (int i0 = 0; i0 < PN / 4; i0 += 8) {
        int page[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {                     // eight page lookups in flight together
          const int j = j0 + rbase + 4 * (i0 + i);
          const int pg = p.page_shift >= 0 ? (j >> p.page_shift) : j / p.page_size;
          page[i] = j < kv_len ? __ldg(bt + pg) : -1;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rbase + 4 * (i0 + i);
          const int j = j0 + r;
          const int off = p.page_shift >= 0 ? (j & (p.page_size - 1)) : j % p.page_size;
          const bool valid = page[i] >= 0;
          const size_t src = valid ? ((((size_t)page[i] * p.nkv + kvh) * p.page_size + off) * HD + ch * 8) : 0;
          const uint32_t dst = (uint32_t)(r * 128 + ((ch ^ (r & 7)) << 4));
#pragma unroll
          for (int a = 0; a < C::HA; ++a) {
            cp_async16z(kd + dst + (uint32_t)(a * C::ATOM_KEYS), p.kc + src + a * 64, valid);
            cp_async16z(vd + dst + (uint32_t)(a * C::ATOM_KEYS), p.vc + src + a * 64, valid);
          }
        }
      }
      cp_async_commit();
      cp_async_wait<0>();                                 // the tile has landed
      fence_proxy_async();                                // for the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[s]);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ the PV products (one thread); without
    // TMA the loaders are all busy and this thread issues S as well, three steps ahead
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      if (!TMA)
        for (int k = 0; k < SB && k < n_steps && ok; ++k) issue_s(k, ok);
      for (int k = 0; k < n_steps && ok; ++k) {
        issue_pv(k, ok);
        if (!TMA && ok && k + SB < n_steps) issue_s(k + SB, ok);
      }
      // nothing of this item may still be on its way to a barrier when the next item sets them up again
      for (int t = max(0, n_tiles - NST); t < n_tiles && ok; ++t)
        if (!mbar_wait(&kv_empty[t % NST], (uint32_t)(t / NST) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 26, t); ok = false;
        }
    }
  }
  } else {
  if (n_t[(warp - SOFTMAX_WARP0) >> 2] > 0) {
    // ------------------------------------------------------------ softmax warps: one thread per row
    const int g = (warp - SOFTMAX_WARP0) >> 2;           // the row tile
    const int n_mine = n_t[g];
    const int quad = warp & 3;                            // the TMEM lanes this warp may read: 32 quad ...
    const int r = quad * 32 + lane;
    const int row = (tile0 + g) * PM + r;
    const bool valid = row < rows_total;
    const int tok = valid ? row / G : 0, head = kvh * G + (valid ? row % G : 0);
    const int pos = kv_len - q_len + tok;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    if (TMA) {
      // this thread's own row of Q into the A-operand layout (rows beyond the sequence zero), while the
      // first K and V tiles are on their way
      const bf16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)head * HD;
      const uint32_t drow = q_s + (uint32_t)(g * C::Q_BYTES + r * 128);
#pragma unroll
      for (int a = 0; a < C::HA; ++a)
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          cp_async16z(drow + (uint32_t)(a * C::ATOM_ROWS) + (uint32_t)((ch ^ (r & 7)) << 4), src + a * 64 + ch * 8, valid);
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full);
    }
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t pv_addr = lane_addr + C::O_COL + (uint32_t)g * HD;
    const uint32_t prow = p_s + (uint32_t)g * C::P_BYTES + (uint32_t)(r * 128);
    constexpr int NC = PN / 32;                           // the row's scores come 32 at a time
    const float sl = p.scale_log2e;
    float m = -INFINITY, l = 0.f;       // m: what the exponentials are taken against, up to 2^8 behind the true maximum
    bool ok = true;

    auto wait_on = [&](uint64_t* bar, uint32_t parity, int role, int t) -> bool {
      bool got = mbar_wait(bar, parity, &abort_flag);
      if (!got) { abort_flag = 1; record_failure(p.err, role, t); }
      return __all_sync(0xffffffffu, got);
    };

    for (int t = 0; t < n_mine; ++t) {
      const int j0 = kv_begin + t * PN;
      const int k = t < n_both ? 2 * t + g : 2 * n_both + (t - n_both);
      const uint32_t s_addr = lane_addr + C::S_COL + (uint32_t)(k % SB) * PN;   // this step's S accumulator
      if (!wait_on(&s_full[k % SB], (uint32_t)(k / SB) & 1u, 24, t)) { ok = false; break; }
      tc_fence_after();
      // ---- the row's PN scores, the hidden ones -inf, and their maximum
      uint32_t v[NC][32];
#pragma unroll
      for (int c = 0; c < NC; ++c) tmem_ld32(s_addr + 32 * c, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[k % SB]);        // the accumulator may take the scores of step k + 3
      if (!valid || j0 + PN - 1 > pos || j0 < lo) {        // some key is hidden from this row
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int j = j0 + 32 * c + i;
            if (!(valid && j <= pos && j >= lo)) v[c][i] = 0xff800000u;
          }
      }
      float mq[NC];                                       // chains side by side, not one of 64 links
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        mq[c] = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) mq[c] = fmax3(mq[c], __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
      }
      float mx = mq[0];
#pragma unroll
      for (int c = 1; c < NC; ++c) mx = fmaxf(mx, mq[c]);
      const float cand = fmaxf(m, mx * sl);               // the scale is positive: it commutes with max
      const bool move = cand > m + 8.f;                   // also the first visible key (m = -inf)
      float corr = 1.f;
      if (move) { corr = fast_exp2(m - cand); m = cand; l *= corr; }      // exp2(-inf) = 0
      if (t > 0) {
        // the PV of the tile before is complete: P may be written again, the output may be touched
        if (!wait_on(&pv_full[g], (uint32_t)(t - 1) & 1u, 25, t)) { ok = false; break; }
        if (__any_sync(0xffffffffu, move)) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 16; ++c) {
            uint32_t ov[16];
            tmem_ld16(pv_addr + 16 * c, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
            tmem_st16(pv_addr + 16 * c, ov);
          }
          tmem_st_wait();
        }
      }
      // ---- exponentials, their sum, P as bf16 into the A-operand layout
      const float use = (m == -INFINITY) ? 0.f : m;
      float lq[8];                                        // partial sums side by side, added up in a fixed order
#pragma unroll
      for (int i = 0; i < 8; ++i) lq[i] = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const uint32_t base = prow + (uint32_t)(c >> 1) * C::ATOM_ROWS;    // an atom of 64 keys
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {                  // 8 keys = one 16-byte chunk
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            e[i] = fast_exp2(fmaf(__uint_as_float(v[c][8 * q8 + i]), sl, -use));      // hidden keys hold -inf: 0
            lq[i] += e[i];
          }
          const int ch = (c & 1) * 4 + q8;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + (uint32_t)((ch ^ (r & 7)) << 4)),
                       "r"(pack_bf16(e[0], e[1])), "r"(pack_bf16(e[2], e[3])), "r"(pack_bf16(e[4], e[5])),
                       "r"(pack_bf16(e[6], e[7])) : "memory");
        }
      }
      tc_fence_before();
      fence_proxy_async();                                // P is read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[g]);
      l += ((lq[0] + lq[1]) + (lq[2] + lq[3])) + ((lq[4] + lq[5]) + (lq[6] + lq[7]));
    }
    if (ok && wait_on(&pv_full[g], (uint32_t)(n_mine - 1) & 1u, 25, n_mine)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(q0 + tok) * p.out_stride + (size_t)head * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ov[32];
        tmem_ld32(pv_addr + 32 * c, ov);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + 32 * c + i) = w;
          }
        }
      }
      tc_fence_before();
    }
  } else if (TMA) {
    if (lane == 0) mbar_arrive(&q_full);                  // a row tile beyond the sequence's rows: nothing to bring
  }
  }
  }   // items
  };
  if (warp < SOFTMAX_WARP0) {
    regs_give_up<REGS_LOW>();
    walk(std::false_type{});
  } else {
    regs_take<REGS_HIGH>();
    walk(std::true_type{});
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---- tensor maps over the caches (they live as long as the process, like the caches' addresses)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;
struct MapKey {
  const void* p; long long planes; int page_size, hd;
  bool operator==(const MapKey& o) const { return p == o.p && planes == o.planes && page_size == o.page_size && hd == o.hd; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.planes * 2654435761LL + k.page_size * 257 + k.hd) << 1);
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;

// cache [planes = pages * kv heads][page_size][hd] bf16; a copy brings 64 values of box_rows keys of one plane
int cache_map(CUtensorMap* out, const void* ptr, long long planes, int page_size, int hd, int box_rows) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
      cudaGetLastError();
      return -5;
    }
    g_encode = (EncodeTiledFn)fn;
  }
  MapKey key{ptr, planes, page_size, hd};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)page_size, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)page_size * hd * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -5;
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

template <int HD, bool TMA>
int launch_pf(const CUtensorMap& mk, const CUtensorMap& mv, const PfParams& p, int ctas, cudaStream_t s) {
  static bool configured[64] = {};
  if (allow_dynamic_smem(attn_prefill_tc_kernel<HD, TMA>, Shape<HD>::SMEM_BYTES, configured)) return -5;
  return launch_ex(attn_prefill_tc_kernel<HD, TMA>, dim3(ctas), dim3(THREADS), Shape<HD>::SMEM_BYTES, s, 1, mk, mv, p);
}

}  // namespace

// q: [T, ...] bf16 rows with stride q_stride, head h at h*hd; out likewise (16-byte aligned rows).
// kcache / vcache: [num_pages][nkv][page_size][hd] bf16. cu_q [S+1], kv_lens [S], block_table [S, bt_stride].
// max_q_len: the longest portion in the batch (sizes the list of work items). Head sizes 64 and 128.
// sm_count: CTAs to launch at most (0: asked from the device).
RLLM_API int rllm_attention_prefill_tc(const void* q, int q_stride, const void* kcache, const void* vcache,
                                       void* out, int out_stride, const int* cu_q, const int* kv_lens,
                                       const int* block_table, int bt_stride, int num_seqs, int max_q_len,
                                       int num_pages, int nh, int nkv, int hd, int page_size, float scale, int window,
                                       int* err, int sm_count, void* stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || page_size <= 0 || num_pages <= 0) return ERR_BAD_SIZE;
  if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return ERR_BAD_ALIGN;
  PfParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.kc = (const bf16*)kcache; p.vc = (const bf16*)vcache;
  p.out = (bf16*)out; p.out_stride = out_stride; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.block_table = block_table; p.bt_stride = bt_stride; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
  p.page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) { p.page_shift = 0; while ((1 << p.page_shift) < page_size) ++p.page_shift; }
  p.window = window; p.scale_log2e = scale * 1.4426950408889634f; p.err = err;
  const int G = nh / nkv;
  p.row_pairs = (max_q_len * G + RT * PM - 1) / (RT * PM); p.num_seqs = num_seqs;
  const long long items = (long long)p.row_pairs * nkv * num_seqs;
  if (items > 2147483647LL) return ERR_TOO_LARGE;
  int sms = sm_count;
  if (sms <= 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return -5;
    }
  }
  const int ctas = items < sms ? (int)items : sms;
  // pages of a power of two from 8 keys up (whole 1 KB swizzle atoms) come by tensor copies
  const bool tma = p.page_shift >= 3 && (long long)num_pages * nkv <= 2147483647LL;
  CUtensorMap mk, mv;
  cudaStream_t s = (cudaStream_t)stream;
  if (tma) {
    const int pn = hd == 64 ? Shape<64>::PN : Shape<128>::PN;
    p.box_rows = page_size < pn ? page_size : pn;
    int rc;
    if ((rc = cache_map(&mk, kcache, (long long)num_pages * nkv, page_size, hd, p.box_rows))) return rc;
    if ((rc = cache_map(&mv, vcache, (long long)num_pages * nkv, page_size, hd, p.box_rows))) return rc;
    return hd == 64 ? launch_pf<64, true>(mk, mv, p, ctas, s) : launch_pf<128, true>(mk, mv, p, ctas, s);
  }
  p.box_rows = 0;
  memset(&mk, 0, sizeof(mk));
  mv = mk;
  return hd == 64 ? launch_pf<64, false>(mk, mv, p, ctas, s) : launch_pf<128, false>(mk, mv, p, ctas, s);
}
