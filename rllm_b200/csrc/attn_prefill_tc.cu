// Prefill attention over the paged bfloat16 cache on the 5th-generation tensor cores (tcgen05),
// head size 64: both products of a tile run as UMMA with their accumulators in TMEM.
//
// A work item is 128 rows, (query token, query head) pairs of ONE kv head (row r of a sequence is
// token r / G, head kvh*G + r % G, as in the mma.sync kernel), and walks the keys the rows can
// see in tiles of 128:
//   warps 0..3  fetch the Q rows once and the K and V tiles through the block table into 128-byte
//               swizzled shared memory, four stages. Pages of a power of two from 8 keys up come
//               by TMA, one copy per page (or per 128 keys of a larger page) and cache, issued by
//               warp 0 alone and counted by the stage's mbarrier; any other page size comes by
//               16-byte cp.async, the four warps taking turns tile by tile, one stage each;
//   warp 4      one thread issues the products:  S = Q K^T  (M 128, N 128 keys, K 64) into one of
//               two S accumulators, and  PV = P V  (M 128, N 64, K 128 keys) with P read from
//               shared memory and V as it lies in the cache tile (an MN-major operand: the
//               contraction runs over key rows);
//   warps 5..12 two threads per row (64 keys of the tile and 32 output values each): read S from
//               TMEM, keep the running maximum and sum in float with exp2, write P as bf16 in
//               the swizzled layout of an A operand, and add the tile's PV (read from TMEM) into
//               the row's output values in registers, rescaled when the maximum moved.
// S of tile t + 1 is computed while the softmax of tile t runs (two S and two PV accumulators,
// 384 TMEM columns). A key j is visible when j <= position of the row and j > position - window.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:573-618 and :328-388 of the reference (scale,
// softmax with the maximum subtracted, weighted V, head h -> kv head h / G, window); unlike the
// reference's prefill kernel a portion also sees what earlier steps left in the cache.
// Every mbarrier wait is bounded; a wait that runs out records an error word and the CTA leaves
// in an orderly way (copies drained, TMEM freed).
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>
#include <unordered_map>

using namespace rllm;
using namespace sm100;

namespace {

constexpr int PM = 128;          // rows per CTA
constexpr int PN = 128;          // keys per tile
constexpr int HD = 64;
constexpr int LOADERS = 4;       // loader warps
constexpr int MMA_WARP = LOADERS;
#ifndef PF_SPLIT
#define PF_SPLIT 2
#endif
constexpr int SPLIT = PF_SPLIT;  // softmax warps per TMEM lane quadrant: each takes 128 / SPLIT keys of a tile
constexpr int KT = PN / SPLIT;   // keys per softmax thread and tile
constexpr int OD = HD / SPLIT;   // output values per softmax thread
constexpr int SOFTMAX_WARP0 = LOADERS + 1;
constexpr int THREADS = (LOADERS + 1 + 4 * SPLIT) * 32;   // warps 0..3 load, warp 4 issues the products, the rest softmax
constexpr int TILE_BYTES = PN * HD * 2;          // 16 KB: one K or V tile, and Q
constexpr int P_BYTES = PM * PN * 2;             // 32 KB: two 64-key sub-tiles of 16 KB
constexpr int KVS = LOADERS;     // K/V stages: loader warp w always fills stage w (tiles w, w + KVS, ...), so its
                                 // waits on that stage's barriers follow one another phase by phase; a warp
                                 // that moved between stages could be two phases ahead, which a parity cannot tell
constexpr int SMEM_BYTES = 1024 + TILE_BYTES * (1 + 2 * KVS) + 2 * P_BYTES;    // Q, K[KVS], V[KVS], P[2]
constexpr int TMEM_COLS = 512;   // S[2] x 128 + PV[2] x 64 = 384
constexpr int S_COL = 0, PV_COL = 256;

struct PfParams {
  const bf16* q; int q_stride;
  const bf16* kc; const bf16* vc;
  bf16* out; int out_stride;
  const int* cu_q; const int* kv_lens; const int* block_table; int bt_stride;
  int nh, nkv, page_size, page_shift, window;
  int box_rows;          // TMA variant: keys per copy = min(page size, 128)
  int row_tiles, num_seqs, sm_count;
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

// TMA: the K and V tiles come by tensor copies over the caches seen as [pages * kv heads][page size][64].
template <bool TMA>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const PfParams p) {
  extern __shared__ uint8_t pf_smem_raw[];
  __shared__ __align__(8) uint64_t kv_full[KVS], kv_empty[KVS], s_full[2], p_full[2], pv_full[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int pair_fail[4];       // a wait of one of a quadrant's two warps ran out: both leave together
  __shared__ float xmax[SPLIT][PM];      // what the two warps of a lane quadrant tell each other (maximum, sum)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)pf_smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_u32(smem);
  const uint32_t k_s = q_s + TILE_BYTES, v_s = k_s + KVS * TILE_BYTES, p_s = v_s + KVS * TILE_BYTES;

  const int G = p.nh / p.nkv;
  if (threadIdx.x == 0) abort_flag = 0;
  if (TMA) {
    // A copy brings whole pages: rows past a sequence's last key keep what the stage held before.
    // The scores of such keys are masked, and their weights are exact zeros, but zero times what
    // an earlier kernel left here need not be zero: start from zeros (later leftovers are keys).
    if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_k); prefetch_tensormap(&tmap_v); }
    uint4* kv = reinterpret_cast<uint4*>(smem + TILE_BYTES);
    for (int i = threadIdx.x; i < 2 * KVS * TILE_BYTES / 16; i += THREADS) kv[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&tmem_base_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch();
  pdl_wait();                                           // q and the newest keys come from the kernel before
  const uint32_t tmem_base = tmem_base_slot;

  // The CTAs (one per SM) share the (row tile, kv head, sequence) items out among themselves:
  // items are numbered from the row tiles that see the most keys down, and round r gives CTA c
  // item r * C + c, or r * C + (C - 1 - c) in odd rounds, so that every CTA gets a like share of
  // long and short ones.
  const int items = p.row_tiles * p.nkv * p.num_seqs;
  for (int round = 0;; ++round) {
  const int item = round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  if (item >= items) break;
  const int tile = p.row_tiles - 1 - item / (p.nkv * p.num_seqs);
  const int kvh = item % p.nkv, seq = (item / p.nkv) % p.num_seqs;
  __syncthreads();                                      // everybody has left the item before
  if (threadIdx.x == 0) {
    for (int i = 0; i < KVS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4 * SPLIT); mbar_init(&pv_full[i], 1); }
    for (int i = 0; i < 4; ++i) pair_fail[i] = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (abort_flag) break;                                // a wait ran out in an earlier item: the kernel's output is void anyway

  const int q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q0;
  const int kv_len = p.kv_lens[seq];
  const int rows_total = q_len * G;
  const bool cta_active = tile * PM < rows_total;       // uniform: an item beyond the sequence's rows is empty
  // keys this item's rows can see at all
  const int tok_first = (tile * PM) / G;
  const int tok_last = min(q_len - 1, (tile * PM + PM - 1) / G);
  const int p_min = kv_len - q_len + tok_first, p_max = kv_len - q_len + tok_last;
  int kv_begin = (p.window > 0 && p_min - p.window + 1 > 0) ? p_min - p.window + 1 : 0;
  kv_begin = kv_begin / PN * PN;
  const int n_tiles = cta_active ? (p_max + 1 - kv_begin + PN - 1) / PN : 0;

  if (warp < LOADERS && TMA) {
    // ------------------------------------------------------------ loader (TMA): warp 0 alone, tile after tile.
    // Lane c looks up the page of the tile's c-th copy; lane 0 tells the stage's barrier how many
    // bytes are coming; every lane with a page issues its two copies. Nothing waits for a tile to
    // land: up to KVS tiles are on their way.
    if (warp == 0) {
      const int* bt = p.block_table + (size_t)seq * p.bt_stride;
      const int copies = PN / p.box_rows;                  // per tile and cache
      const uint32_t copy_bytes = (uint32_t)p.box_rows * HD * 2;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % KVS;
        if (t >= KVS) {
          int w_ok = 1;
          if (lane == 0 && !mbar_wait(&kv_empty[s], (uint32_t)(t / KVS - 1) & 1u, &abort_flag)) {
            abort_flag = 1; record_failure(p.err, 21, t); w_ok = 0;
          }
          if (__shfl_sync(0xffffffffu, w_ok, 0) == 0) break;
        }
        if (t == 0) {
          // the Q rows of the CTA, rows beyond the sequence zero; landed before the first tile is announced
          const int ch = lane & 7, rbase = lane >> 3;
#pragma unroll 4
          for (int i = 0; i < 32; ++i) {
            const int r = rbase + 4 * i;
            const int row = tile * PM + r;
            const bool valid = row < rows_total;
            const int tok = valid ? row / G : 0, head = kvh * G + (valid ? row % G : 0);
            const bf16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)head * HD + ch * 8;
            cp_async16z(q_s + (uint32_t)(r * 128 + ((ch ^ (r & 7)) << 4)), src, valid);
          }
          cp_async_commit();
          cp_async_wait<0>();
          fence_proxy_async();
          __syncwarp();
        }
        const int j = kv_begin + t * PN + lane * p.box_rows;            // first key of this lane's copy
        const bool mine = lane < copies && j < kv_len;
        const int page = mine ? __ldg(bt + (j >> p.page_shift)) : 0;
        const uint32_t n = __popc(__ballot_sync(0xffffffffu, mine));
        if (lane == 0) mbar_expect_tx(&kv_full[s], 2 * n * copy_bytes);
        __syncwarp();
        if (mine) {
          const uint32_t dst = (uint32_t)s * TILE_BYTES + (uint32_t)lane * copy_bytes;
          const int off = j & (p.page_size - 1);
          tma_load_3d(k_s + dst, &tmap_k, &kv_full[s], 0, off, page * p.nkv + kvh);
          tma_load_3d(v_s + dst, &tmap_v, &kv_full[s], 0, off, page * p.nkv + kvh);
        }
      }
    }
  } else if (warp < LOADERS) {
    // ------------------------------------------------------------ loaders: warp w fetches the tiles w, w + 4, ...
    // whole, waits until they have landed and announces them at once, so a tile is ready long
    // before its turn (up to KVS tiles are on the way, from different warps).
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;
    const int ch = lane & 7;                              // this lane's 16-byte chunk of a 128-byte row
    const int rbase = lane >> 3;                          // its rows: rbase + 4 i, i < 32
    for (int t = warp; t < n_tiles; t += LOADERS) {
      const int s = t % KVS;
      if (t >= KVS) {
        int w_ok = 1;
        if (lane == 0 && !mbar_wait(&kv_empty[s], (uint32_t)(t / KVS - 1) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 21, t); w_ok = 0;
        }
        if (__shfl_sync(0xffffffffu, w_ok, 0) == 0) break;
      }
      if (t == 0) {
        // the Q rows of the CTA, rows beyond the sequence zero
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int r = rbase + 4 * i;
          const int row = tile * PM + r;
          const bool valid = row < rows_total;
          const int tok = valid ? row / G : 0, head = kvh * G + (valid ? row % G : 0);
          const bf16* src = p.q + (size_t)(q0 + tok) * p.q_stride + (size_t)head * HD + ch * 8;
          cp_async16z(q_s + (uint32_t)(r * 128 + ((ch ^ (r & 7)) << 4)), src, valid);
        }
      }
      const int j0 = kv_begin + t * PN;
      const uint32_t kd = k_s + (uint32_t)s * TILE_BYTES, vd = v_s + (uint32_t)s * TILE_BYTES;
#pragma unroll 1
      for (int i0 = 0; i0 < 32; i0 += 8) {
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
          cp_async16z(kd + dst, p.kc + src, valid);
          cp_async16z(vd + dst, p.vc + src, valid);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();                                 // the tile has landed
      fence_proxy_async();                                // for the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[s]);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ the products (one thread)
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t id_s = idesc(PM, PN, false);
      constexpr uint32_t id_pv = idesc(PM, HD, true);
      bool ok = true;
      auto issue_s = [&](int t) {
        const int s = t & 1, ks = t % KVS;
        if (!mbar_wait(&kv_full[ks], (uint32_t)(t / KVS) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 22, t); ok = false; return;
        }
        tc_fence_after();
        const uint64_t dq = umma_desc_sw128(q_s), dk = umma_desc_sw128(k_s + (uint32_t)ks * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(tmem_base + S_COL + (uint32_t)s * PN, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), id_s, k > 0);
        umma_commit(&s_full[s]);
      };
      issue_s(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t & 1;
        if (t + 1 < n_tiles) issue_s(t + 1);            // the next scores while this tile's softmax runs
        if (!ok) break;
        if (!mbar_wait(&p_full[s], (uint32_t)(t >> 1) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 23, t); ok = false; break;
        }
        tc_fence_after();
        const uint32_t pa = p_s + (uint32_t)s * P_BYTES, va = v_s + (uint32_t)(t % KVS) * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < PN / 16; ++ks) {
          // P: K-major, two 64-key sub-tiles of 16 KB; V: MN-major, 16 key rows = 2 KB per step
          const uint64_t dp = umma_desc_sw128(pa + (uint32_t)(ks >> 2) * TILE_BYTES) + (uint64_t)((ks & 3) * 2);
          const uint64_t dv = umma_desc_sw128(va + (uint32_t)ks * 2048u);
          umma_bf16(tmem_base + PV_COL + (uint32_t)s * HD, dp, dv, id_pv, ks > 0);
        }
        umma_commit(&kv_empty[t % KVS]);                // K and V of this stage are read
        umma_commit(&pv_full[s]);
      }
      // nothing of this item may still be on its way to a barrier when the next item sets them up again
      for (int t = max(0, n_tiles - KVS); t < n_tiles && ok; ++t)
        if (!mbar_wait(&kv_empty[t % KVS], (uint32_t)(t / KVS) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 26, t); ok = false;
        }
    }
  } else if (n_tiles > 0) {
    // ------------------------------------------------------------ softmax warps
    // SPLIT warps share each TMEM lane quadrant (a warp may only read the 32 lanes of its index
    // mod 4): warps w, w + 4, ... serve the same 32 rows, each KT keys of a tile and OD of the 64
    // output values. They agree on the row's maximum through shared memory; each keeps the sum
    // of its own exponentials, added at the end. More warps per quadrant hide the TMEM latency.
    const int quad = warp & 3;
    const int half = (warp - SOFTMAX_WARP0) >> 2;       // which KT keys of a tile, which OD output values
    const int r = quad * 32 + lane;
    const int row = tile * PM + r;
    const bool valid = row < rows_total;
    const int tok = valid ? row / G : 0, head = kvh * G + (valid ? row % G : 0);
    const int pos = kv_len - q_len + tok;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float sl = p.scale_log2e;
    float o[OD];
#pragma unroll
    for (int i = 0; i < OD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f, corr_prev = 1.f;
    bool ok = true;
    auto pair_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + quad), "n"(32 * SPLIT) : "memory"); };

    auto add_pv = [&](int t, float corr) {              // O = O * corr + PV(t), this thread's 32 values
      const int s = t & 1;
      bool got = mbar_wait(&pv_full[s], (uint32_t)(t >> 1) & 1u, &abort_flag);
      if (!got) { abort_flag = 1; record_failure(p.err, 25, t); }
      got = __all_sync(0xffffffffu, got);
      if (!got) { ok = false; return; }
      tc_fence_after();
      uint32_t v[OD / 16][16];
#pragma unroll
      for (int q2 = 0; q2 < OD / 16; ++q2) tmem_ld16(lane_addr + PV_COL + (uint32_t)s * HD + half * OD + 16 * q2, v[q2]);
      tmem_ld_wait();
#pragma unroll
      for (int q2 = 0; q2 < OD / 16; ++q2)
#pragma unroll
        for (int i = 0; i < 16; ++i) o[16 * q2 + i] = fmaf(o[16 * q2 + i], corr, __uint_as_float(v[q2][i]));
      tc_fence_before();
    };

    for (int t = 0; t < n_tiles; ++t) {
      const int s = t & 1;
      const int j0 = kv_begin + t * PN + half * KT;       // first key of this thread's KT
      if (ok) {
        bool got = mbar_wait(&s_full[s], (uint32_t)(t >> 1) & 1u, &abort_flag);
        if (!got) { abort_flag = 1; record_failure(p.err, 24, t); }
        got = __all_sync(0xffffffffu, got);
        if (!got) ok = false;
      }
      if (!ok) pair_fail[quad] = 1;
      // ---- this thread's KT scores, read once
      constexpr int NQ = KT / 16;
      uint32_t v[NQ][16];
      if (ok) {
        tc_fence_after();
        const uint32_t s_addr = lane_addr + S_COL + (uint32_t)s * PN + half * KT;
#pragma unroll
        for (int q4 = 0; q4 < NQ; ++q4) tmem_ld16(s_addr + 16 * q4, v[q4]);
        tmem_ld_wait();
      }
      const bool edge = !valid || j0 + KT - 1 > pos || j0 < lo;      // some key is hidden from this row
      float mx = -INFINITY;
      if (ok) {
        if (edge) {
#pragma unroll
          for (int q4 = 0; q4 < NQ; ++q4)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int j = j0 + 16 * q4 + i;
              if (!(valid && j <= pos && j >= lo)) v[q4][i] = 0xff800000u;      // -inf
            }
        }
#pragma unroll
        for (int q4 = 0; q4 < NQ; ++q4)
#pragma unroll
          for (int i = 0; i < 16; ++i) mx = fmaxf(mx, __uint_as_float(v[q4][i]));
      }
      // ---- the row's maximum over both halves (the barrier is met also after a failed wait)
      xmax[half][r] = mx;
      pair_sync();
#pragma unroll
      for (int h2 = 0; h2 < SPLIT; ++h2) mx = fmaxf(mx, xmax[h2][r]);
      const bool leave = pair_fail[quad] != 0;
      pair_sync();                                        // both have read before the next tile writes
      if (leave) { ok = false; break; }
      const float m_new = fmaxf(m, mx * sl);              // the scale is positive: it commutes with max
      const float use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = fast_exp2(m - use);              // exp2(-inf) = 0
      m = m_new;
      l *= corr;
      // ---- exponentials, their sum, P as bf16 into the A-operand layout (64-key sub-tiles of 16 KB)
      const int kc0 = half * KT;                          // first key column of this thread within the tile
      const uint32_t prow = p_s + (uint32_t)s * P_BYTES + (uint32_t)(kc0 >> 6) * TILE_BYTES + (uint32_t)(r * 128);
#pragma unroll
      for (int q4 = 0; q4 < NQ; ++q4) {
        float e[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          e[i] = fast_exp2(fmaf(__uint_as_float(v[q4][i]), sl, -use));     // hidden keys hold -inf: 0
          l += e[i];
        }
        const int ch = ((kc0 & 63) >> 3) + 2 * q4;        // first of two 16-byte chunks
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)(((ch) ^ (r & 7)) << 4)),
                     "r"(pack_bf16(e[0], e[1])), "r"(pack_bf16(e[2], e[3])), "r"(pack_bf16(e[4], e[5])),
                     "r"(pack_bf16(e[6], e[7])) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)(((ch + 1) ^ (r & 7)) << 4)),
                     "r"(pack_bf16(e[8], e[9])), "r"(pack_bf16(e[10], e[11])), "r"(pack_bf16(e[12], e[13])),
                     "r"(pack_bf16(e[14], e[15])) : "memory");
      }
      tc_fence_before();
      fence_proxy_async();                                // P is read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
      // ---- the tile before this one: its PV is ready by now; fold it into the row's output
      if (t > 0) add_pv(t - 1, corr_prev);
      corr_prev = corr;
    }
    if (ok) add_pv(n_tiles - 1, corr_prev);             // every tile's PV entered with its own tile's factor
    // ---- the two halves' sums of exponentials meet (met also after a failed wait)
    xmax[half][r] = l;
    pair_sync();
    l = 0.f;
#pragma unroll
    for (int h2 = 0; h2 < SPLIT; ++h2) l += xmax[h2][r];       // the same order in every thread of the row
    if (ok && valid) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(q0 + tok) * p.out_stride + (size_t)head * HD + half * OD;
#pragma unroll
      for (int c = 0; c < OD; c += 8) {
        uint4 w;
        w.x = pack_bf16(o[c] * inv, o[c + 1] * inv); w.y = pack_bf16(o[c + 2] * inv, o[c + 3] * inv);
        w.z = pack_bf16(o[c + 4] * inv, o[c + 5] * inv); w.w = pack_bf16(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = w;
      }
    }
  }
  }   // items
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
  const void* p; long long planes; int page_size;
  bool operator==(const MapKey& o) const { return p == o.p && planes == o.planes && page_size == o.page_size; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.planes * 2654435761LL + k.page_size) << 1);
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;

// cache [planes = pages * kv heads][page_size][64] bf16; a copy brings box_rows keys of one plane
int cache_map(CUtensorMap* out, const void* ptr, long long planes, int page_size, int box_rows) {
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
  MapKey key{ptr, planes, page_size};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)page_size, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)page_size * HD * 2};
    cuuint32_t box[3] = {(cuuint32_t)HD, (cuuint32_t)box_rows, 1};
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

template <bool TMA>
int launch_pf(const CUtensorMap& mk, const CUtensorMap& mv, const PfParams& p, int ctas, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel<TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess) { cudaGetLastError(); return -5; }
    configured = true;
  }
  return launch_ex(attn_prefill_tc_kernel<TMA>, dim3(ctas), dim3(THREADS), SMEM_BYTES, s, 1, mk, mv, p);
}

}  // namespace

// q: [T, ...] bf16 rows with stride q_stride, head h at h*64; out likewise (16-byte aligned rows).
// kcache / vcache: [num_pages][nkv][page_size][64] bf16. cu_q [S+1], kv_lens [S], block_table [S, bt_stride].
// max_q_len: the longest portion in the batch (sizes the list of work items). Head size 64 only.
// sm_count: CTAs to launch at most (0: asked from the device).
RLLM_API int rllm_attention_prefill_tc(const void* q, int q_stride, const void* kcache, const void* vcache,
                                       void* out, int out_stride, const int* cu_q, const int* kv_lens,
                                       const int* block_table, int bt_stride, int num_seqs, int max_q_len,
                                       int num_pages, int nh, int nkv, int hd, int page_size, float scale, int window,
                                       int* err, int sm_count, void* stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (hd != HD || nkv <= 0 || nh % nkv || page_size <= 0 || num_pages <= 0) return ERR_BAD_SIZE;
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
  p.row_tiles = (max_q_len * G + PM - 1) / PM; p.num_seqs = num_seqs;
  const long long items = (long long)p.row_tiles * nkv * num_seqs;
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
  if (tma) {
    p.box_rows = page_size < PN ? page_size : PN;
    int rc;
    if ((rc = cache_map(&mk, kcache, (long long)num_pages * nkv, page_size, p.box_rows))) return rc;
    if ((rc = cache_map(&mv, vcache, (long long)num_pages * nkv, page_size, p.box_rows))) return rc;
    return launch_pf<true>(mk, mv, p, ctas, (cudaStream_t)stream);
  }
  p.box_rows = 0;
  memset(&mk, 0, sizeof(mk));
  mv = mk;
  return launch_pf<false>(mk, mv, p, ctas, (cudaStream_t)stream);
}
