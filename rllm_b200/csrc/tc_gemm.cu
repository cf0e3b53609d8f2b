// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), operands staged by
// TMA, accumulators in TMEM:
//     C[T, N] = X[T, K] * W[N, K]^T          (X activations, W weights as stored, both K-major)
//
// The weight tile is the MMA's A operand (M = 128 weight rows) and the token tile is its B
// operand (N = BN tokens), so a decode step with a handful of tokens still fills the 128-row MMA
// and streams every weight byte exactly once. Steps of up to 64 tokens (128 for a narrow weight)
// run token tiles of 16 or 32 in the first kernel below; more tokens run in the persistent kernel
// further down, whose token tile is any multiple of 16 up to 256 (128 with the gate/up pair),
// chosen so that the tiles fill whole waves of CTAs. The accumulator D[weight row (TMEM lane),
// token (TMEM column)] is read back with tcgen05.ld by the epilogue warps, thread = weight row, and
// written as C[token][row]. Gate/up pairs of 33 tokens and more (with no norm in front) exchange the
// roles: tokens on the accumulator's rows, the tile's 128 gate and 128 up weight rows one operand of
// 256 columns; 64 + 64 rows where tiles of 128 would leave most SMs without one (up to 128 tokens
// against 8,192 features).
//
// One CTA = one 128 x BN output tile over a range of K: warp 0 issues TMA loads into a ring of
// shared-memory stages, warp 1 issues the MMAs (one thread) and owns the TMEM allocation,
// warps 2-5 run the epilogue (2-9 in the persistent kernel: one warp alone on a scheduler waits
// out every instruction's latency). The small-tile kernel has a second MMA warp (6), see `Cfg::TWO`.
//
// Fused RMSNorm (NORM variants, steps of up to 64 tokens): X is not read by TMA. The input is the
// float residual stream h and a norm weight g; warps 2-5 build the B operand themselves, stage
// by stage: bf16(h[t,k] * g[k]) written in the 128-byte swizzled layout the MMA expects, while
// they add up h[t,k]^2. Since rsqrt(mean(h^2) + eps) is one number per token it commutes with
// the product and is applied in the epilogue: y[t,n] = rstd[t] * sum_k (h[t,k] g[k]) W[n,k].
// A list of row indices lets the product read chosen rows of h only (the output head).
//
// Split-K for small batches (few output tiles, long K) runs inside a thread-block cluster:
// the CTAs of a cluster share one output tile and take consecutive ranges of K. Rank r owns
// the token columns r, r + C, ...: every rank pushes its float partial column (and its part
// of the sum of squares) into the owner's shared memory through distributed shared memory,
// one cluster barrier later the owner adds the parts in rank order from its own shared memory
// and runs the epilogue. Nothing goes through global memory and the sum does not depend on
// timing. The landing area is a region of its own, so a rank pushes as soon as its own products
// are done; only the gate/up pair at 32 tokens, which that region would leave with two stages,
// lands in the (by then idle) stage ring after one more cluster barrier.
//
// Programmatic dependent launch: the kernel lets its successor start at once, and itself
// fetches its first weight tiles (which no earlier kernel writes) before it waits for its
// predecessor; activations are read and outputs written only after that wait. Small token
// tiles keep their shared memory under half an SM's, so that the successor's CTAs find room
// beside them and their weight tiles are already on the way when the predecessor ends.
//
// Epilogues: store bf16 | store float (logits) | add into the float residual stream |
// SwiGLU over a gate/up pair of weight tiles (two accumulators): out = silu(g) * u |
// rotary position encoding of q and k heads with the write of k and v into the paged cache (in the
// persistent kernel through shared memory, so that a thread moves 8 neighbouring features of a token).
// Reference counterparts: gemm_bf16_tc (src/gpu/cuda/shaders/matmul_tc.cu:224-413, wmma),
// matvec_bf16 (matmul.cu:49-77), fused_gate_up_swiglu_bf16 (moe.cu:86-147), rms_norm
// (rms_norm.cu:78-115), rotary_embedding (rope.cu:62-77) and copy_to_paged_kv_cache
// (attention.cu:295-300).
//
// Every mbarrier wait is bounded; on a time-out the CTA records an error word, drains what it
// has in flight, still meets its cluster's barriers, frees its TMEM and returns.
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>
#include <unordered_map>

using namespace rllm;
using namespace sm100;

namespace {

enum : int { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU = 3, EPI_QKV_ROPE = 4 };

constexpr int BM = 128;        // weight rows per tile (MMA M)
constexpr int BK = 64;         // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;   // warp 0 TMA, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int THREADS_SMALL = 224;   // the small-tile kernel has a second MMA warp (6)
constexpr int THREADS_MANY = 320;    // the persistent kernel has eight epilogue warps (2..9), two on each quarter of the rows
constexpr int MAX_CLUSTER = 8;
// shared memory of a small-tile CTA in KB: 84 + 138 (gate/up pair) = 222 KB, so that any two
// small-tile kernels of a layer fit one SM together (measured: worth 20 % of a step of 9 to 64 tokens)
constexpr int SMALL_KB = 84, SMALL_DUAL_KB = 138;
constexpr int NORM_MAX_TOKENS = 64;
constexpr int NORM_MAX_T = NORM_MAX_TOKENS;        // the fused-norm variants take steps of at most this many tokens

// the most column slots a landing area needs. Tiles of 16: ranks * ceil(BN / ranks) over 1..8
// ranks. Wider tiles are split over 1, 2, 4 or 8 ranks only, each owning a multiple of 4 columns.
constexpr int max_slots(int bn) {
  int m = 0;
  for (int s = 1; s <= MAX_CLUSTER; ++s) {
    if (bn >= 32 && (s & (s - 1))) continue;
    const int per = (bn + s - 1) / s;
    const int v = s * (bn >= 32 ? ((per + 3) & ~3) : per);
    if (v > m) m = v;
  }
  return m;
}

template <int BN, bool DUAL> struct Cfg {
  static constexpr int A_TILES = DUAL ? 2 : 1;
  static constexpr int A_BYTES = BM * BK * 2;                  // 16 KB per weight tile
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
  // token tiles up to 64 (decode, small mixed steps) stay under half an SM's shared memory so
  // that two kernels' CTAs are resident side by side; large tiles take what one CTA can have
  static constexpr bool SMALL = BN <= 64;
  // a landing area of its own only where it leaves an even number of stages (see TWO): tiles of 16 of
  // a single weight tile; the others land in the (by then idle) stage ring
  static constexpr bool DEDICATED = BN <= 16 && !DUAL;
  static constexpr bool VEC = BN >= 32;                        // parts travel four columns at a time
  static constexpr int SLOTS = max_slots(BN);
  static constexpr int LAND_BYTES = SLOTS * A_TILES * BM * 4;
  // 84 KB + 138 KB (gate/up pair) = 222 KB: any two small-tile kernels of a layer fit one SM together
  static constexpr int BUDGET = (SMALL ? (DUAL ? SMALL_DUAL_KB : SMALL_KB) : 200) * 1024 - 1024 - (DEDICATED ? LAND_BYTES : 0);
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = 1024 + RING_BYTES + (DEDICATED ? LAND_BYTES : 0);   // + alignment slack
  // Two MMA-issuing threads take the K blocks in turn, each into an accumulator set of its own,
  // when the stages are even in number: K block i lies in stage i % STAGES, so each stage then
  // belongs to one of the two for good, and a thread that waits for a stage's next filling has
  // itself consumed the filling before. (With an odd number a thread could ask for a stage's
  // second filling before the first, which another thread consumes, has even arrived: TMA copies
  // land in any order, and a parity cannot tell "not yet" from "twice".)
  static constexpr bool TWO = SMALL && STAGES % 2 == 0;
  static constexpr int ACC_COLS = A_TILES * BN;                 // one accumulator set
  static constexpr int ALL_COLS = (TWO ? 2 : 1) * ACC_COLS;
  static constexpr int TMEM_COLS = ALL_COLS <= 32 ? 32 : ALL_COLS <= 64 ? 64 : ALL_COLS <= 128 ? 128
                                   : ALL_COLS <= 256 ? 256 : 512;
  static_assert(DEDICATED || LAND_BYTES <= RING_BYTES, "the landing area must fit in the stage ring");
};

// What the rotary epilogue needs besides the product (see rllm_tc_gemm_qkv_rope).
struct RopeArgs {
  const int* positions;     // [T] absolute position of each token
  const float* inv_freq;    // [rot_dim / 2]
  const float2* cos_sin;    // [T][rot_dim / 2] (cos, sin) of positions[t] * inv_freq[i], or null: computed here
  const int* slots;         // [T] page * page_size + offset, < 0: do not write; may be null
  bf16* kcache;             // [pages][nkv][page_size][hd]
  bf16* vcache;
  int nh, nkv, hd, page_size, rot_dim;
};

// The input of the fused-RMSNorm variants: rows of the float residual stream and the norm weight.
struct NormArgs {
  const float* h;     // [*, K] float, row stride ldh
  long long ldh;
  const int* rows;    // null: token t reads row t; else row rows[t]
  const void* g;      // norm weight [K]
  int g_is_bf16;      // 1: bfloat16, 0: float
  float eps;
};

struct Params {
  void* C;            // output, type by epilogue
  int ldc;            // row stride of C in elements
  int T, N, K;        // tokens, output features, inner size
  int up_row0;        // DUAL: first weight row of the "up" half
  int splits;         // CTAs per cluster = ranges of K
  int bn;             // persistent kernel: tokens per tile (a multiple of 16, at most the template's BN)
  int* err;           // device error word (0 = fine)
  RopeArgs rope;
  NormArgs norm;      // NORM variants only
};

template <int EPI>
__device__ __forceinline__ void emit(const Params& p, int t, int n, float v, float u) {
  const size_t o = (size_t)t * p.ldc + n;
  if (EPI == EPI_STORE) ((bf16*)p.C)[o] = __float2bfloat16_rn(v);
  else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = v;
  else if (EPI == EPI_ACCUM_F32) ((float*)p.C)[o] += v;
  else if (EPI == EPI_SWIGLU) ((bf16*)p.C)[o] = __float2bfloat16_rn(__fdividef(v, 1.f + __expf(-v)) * u);   // float, rounded once to bfloat16
}

// (cos, sin) of a token's angle at one frequency, when the caller gave no table. Not inlined and returned
// by value: sincosf's slow path, copied into an unrolled epilogue loop, is more code than the loop itself,
// and results passed through memory would put the loop's arrays there too. The engine passes a table.
__device__ __noinline__ float2 angle_of(const RopeArgs& r, int t, int i) {
  float sn, cs;
  sincosf((float)r.positions[t] * r.inv_freq[i], &sn, &cs);
  return make_float2(cs, sn);
}

// Rotary epilogue for one (token, output row n) whose pre-rotation value is v and whose pair
// partner's value is w (partner = n +- rot_dim/2 inside the same head). Rows are laid out
// [q heads | k heads | v heads] x hd. q is stored rotated into C; k rotated and v as is go to
// C as well (so the buffer stays complete) and into the paged cache.
__device__ __forceinline__ void emit_rope(const Params& p, int t, int n, float v, float w) {
  const RopeArgs& r = p.rope;
  const int head = n / r.hd, d = n % r.hd;
  float out = v;
  if (head < r.nh + r.nkv && d < r.rot_dim) {
    const int half = r.rot_dim >> 1;
    const int i = d < half ? d : d - half;
    float sn, cs;
    if (r.cos_sin) { const float2 v = r.cos_sin[(size_t)t * half + i]; cs = v.x; sn = v.y; }
    else sincosf((float)r.positions[t] * r.inv_freq[i], &sn, &cs);
    out = d < half ? v * cs - w * sn : w * sn + v * cs;
  }
  const bf16 ob = __float2bfloat16_rn(out);
  ((bf16*)p.C)[(size_t)t * p.ldc + n] = ob;
  if (head >= r.nh && r.slots) {
    const int slot = r.slots[t];
    if (slot >= 0) {
      const int page = slot / r.page_size, off = slot % r.page_size;
      const bool is_k = head < r.nh + r.nkv;
      const int kvh = is_k ? head - r.nh : head - r.nh - r.nkv;
      bf16* dst = (is_k ? r.kcache : r.vcache) + (((size_t)page * r.nkv + kvh) * r.page_size + off) * r.hd;
      dst[d] = ob;
    }
  }
}


__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void epilogue_warps_sync() {       // warps 2..5 only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ void epilogue8_sync() {            // the persistent kernel's warps 2..9
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

template <int BN, int EPI, bool NORM>
__global__ void __launch_bounds__(THREADS_SMALL, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const Params p) {
  constexpr bool DUAL = (EPI == EPI_SWIGLU);
  constexpr bool ROPE = (EPI == EPI_QKV_ROPE);
  typedef Cfg<BN, DUAL> C;
  constexpr int ACCS = C::A_TILES;
  constexpr int W_BYTES = C::A_TILES * C::A_BYTES;
  static_assert(!NORM || BN <= 64, "the fused norm builds token tiles of at most 64 rows");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int never_flag;
  __shared__ float ss_part[NORM ? BN : 1];                 // this rank's sum of h^2 per token of the tile
  __shared__ __align__(16) float ss_land[NORM ? MAX_CLUSTER * BN : 4];   // [rank][slot]: the ranks' parts for the columns owned here

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  // token tiles are the fastest grid index: the CTAs that share a weight tile start together and
  // all but the first find it in L2
  const int n0 = blockIdx.y * BM;          // first weight row / output feature of the tile
  const int t0 = blockIdx.x * BN;          // first token of the tile
  const bool clustered = p.splits > 1;
  const bool landing = clustered || ROPE;  // the epilogue goes through the landing area
  const int rank = clustered ? (int)cluster_rank() : 0;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_begin = (int)((long long)rank * kb_total / p.splits);
  const int kb_end = (int)((long long)(rank + 1) * kb_total / p.splits);
  const int n_kb = kb_end - kb_begin;
  const bool two_sets = C::TWO && n_kb >= 2;       // else the second accumulator set is never written
  // partial columns pushed here by every rank: float [ranks][slots per rank][ACCS][BM] (tiles of 16),
  // float4 [ranks][ACCS][groups of four columns per rank][BM] (wider tiles)
  float* land = reinterpret_cast<float*>(C::DEDICATED ? smem + C::RING_BYTES : smem);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], NORM ? 5 : 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, two_sets ? 2 : 1);         // one arrival per MMA thread that has K blocks
    abort_flag = 0;
    never_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_w); if (!NORM) prefetch_tensormap(&tmap_x); }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch();        // the next kernel may start its prologue: every CTA of this one holds its TMEM by now
  // a landing area of its own may be written as soon as its CTA runs: this arrival says so
  if (clustered && C::DEDICATED) cluster_arrive();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();   // weights are read once per step
      const uint64_t pol_x = policy_evict_last();    // the token tile is shared by every weight tile
      // weights of the first stages do not depend on the kernel before this one
      const int pre = n_kb < C::STAGES ? n_kb : C::STAGES;
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + (size_t)i * C::STAGE_BYTES;
        mbar_expect_tx(&full_bar[i], NORM ? W_BYTES : C::STAGE_BYTES);
        const int k = (kb_begin + i) * BK;
        tma_load_2d_hint(st, &tmap_w, &full_bar[i], k, n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + C::A_BYTES, &tmap_w, &full_bar[i], k, p.up_row0 + n0, pol_w);
      }
      if (!NORM) {
        pdl_wait();                                  // activations come from the kernel before
        for (int i = 0; i < pre; ++i) {
          uint8_t* st = smem + (size_t)i * C::STAGE_BYTES;
          tma_load_2d_hint(st + W_BYTES, &tmap_x, &full_bar[i], (kb_begin + i) * BK, t0, pol_x);
        }
      }
      int issued = pre;
      for (int i = pre; i < n_kb; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag)) { abort_flag = 1; record_failure(p.err, 1); break; }
        uint8_t* st = smem + (size_t)s * C::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], NORM ? W_BYTES : C::STAGE_BYTES);
        const int k = (kb_begin + i) * BK;
        tma_load_2d_hint(st, &tmap_w, &full_bar[s], k, n0, pol_w);
        if (DUAL) tma_load_2d_hint(st + C::A_BYTES, &tmap_w, &full_bar[s], k, p.up_row0 + n0, pol_w);
        if (!NORM) tma_load_2d_hint(st + W_BYTES, &tmap_x, &full_bar[s], k, t0, pol_x);
        issued = i + 1;
      }
      if (abort_flag) {
        // let copies already issued land before the CTA's shared memory is given back
        for (int i = max(0, issued - C::STAGES); i < issued; ++i)
          mbar_wait(&full_bar[i % C::STAGES], (uint32_t)(i / C::STAGES) & 1u, &never_flag, 200000000LL);
      }
    }
  } else if (warp == 1 || (C::TWO && warp == 6)) {
    // ------------------------------------------------------------ MMA issuers
    // Issuing a tcgen05.mma or a commit costs its thread some 50 ns whatever the size, and a token
    // tile of 16 or 32 needs five of them (nine with a gate/up pair) for every K block: one thread
    // would hold the weight stream at about 60 GB/s per SM. With an even number of stages two
    // threads (warps 1 and 6) take the K blocks in turn; the epilogue adds their accumulator sets.
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      constexpr int STEP = C::TWO ? 2 : 1;
      const int w = warp == 1 ? 0 : 1;
      const uint32_t acc_addr = tmem_base + (uint32_t)(w * C::ACC_COLS);
      // a descriptor moves with its address (16 bytes a unit): one is built, the rest are sums
      const uint64_t d0 = umma_desc_sw128(smem_u32(smem));
      bool ok = true;
      for (int i = w; i < n_kb && ok; i += STEP) {
        const int s = i % C::STAGES;
        const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, &abort_flag)) { abort_flag = 1; record_failure(p.err, 2); ok = false; break; }
        tc_fence_after();
        const uint64_t da = d0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
        const uint64_t db = da + (uint64_t)(W_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t acc = (i > w || k > 0) ? 1u : 0u;
          const uint64_t koff = (uint64_t)(k * UMMA_K * 2 / 16);
          umma_bf16(acc_addr, da + koff, db + koff, idesc, acc);
          if (DUAL) umma_bf16(acc_addr + BN, da + (uint64_t)(C::A_BYTES >> 4) + koff, db + koff, idesc, acc);
        }
        umma_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
      }
      if (ok && n_kb > w) umma_commit(&acc_bar);      // this thread's accumulator set is complete
    }
  }
  bool epi_ok = false;
  const int row = (warp & 3) * 32 + lane;         // TMEM lanes [32 (warp & 3), +32) belong to this warp
  const int n = n0 + row;                         // output feature of this thread
  const float inv_k = 1.f / (float)p.K;
  const bool epi_warp = warp >= 2 && warp <= 5;
  // 16 accumulator columns of this thread's row: the sum of the two sets where there are two
  auto ld_acc = [&](uint32_t addr, uint32_t (&v)[16]) {
    tmem_ld16(addr, v);
    if (two_sets) {
      uint32_t w2[16];
      tmem_ld16(addr + (uint32_t)C::ACC_COLS, w2);
      tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) + __uint_as_float(w2[jj]));
    }
  };
  if (epi_warp) {
    // ------------------------------------------------------------ epilogue warps (2..5)
    pdl_wait();                                   // nothing is read or written before the predecessor is done
    if (NORM) {
      // ---- they first build the token operand: bf16(h * g), 128-byte swizzled, and add up h^2
      constexpr int RPT = BN / 16;                // token rows per thread
      const int pt = (warp - 2) * 32 + lane;      // 0..127
      const int j = pt & 7;                       // which 16-byte chunk (8 values of K) of a 64-wide block
      const float* hrow[RPT];
      float ss[RPT];
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int tg = t0 + (pt >> 3) + 16 * r;
        hrow[r] = tg < p.T ? p.norm.h + (size_t)(p.norm.rows ? p.norm.rows[tg] : tg) * p.norm.ldh : nullptr;
        ss[r] = 0.f;
      }
      // The loads of h and g for the next PF stages are always in flight (registers), so that a
      // stage costs a write to shared memory, not a trip to L2.
      constexpr int PF = BN <= 16 ? 4 : 2;
      float4 ha[PF][RPT], hb[PF][RPT];
      uint4 ga[PF], gb[PF];
      auto fetch = [&](int i, float4 (&a)[RPT], float4 (&b)[RPT], uint4& g0, uint4& g1) {
        const int kk = (kb_begin + i) * BK + 8 * j;
        g0 = g1 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < RPT; ++r) a[r] = b[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n_kb && kk < p.K) {               // K is a multiple of 8: a chunk is inside or outside
          if (p.norm.g_is_bf16) {
            g0 = *reinterpret_cast<const uint4*>((const bf16*)p.norm.g + kk);
          } else {
            g0 = *reinterpret_cast<const uint4*>((const float*)p.norm.g + kk);
            g1 = *reinterpret_cast<const uint4*>((const float*)p.norm.g + kk + 4);
          }
#pragma unroll
          for (int r = 0; r < RPT; ++r) {
            if (hrow[r]) {
              a[r] = *reinterpret_cast<const float4*>(hrow[r] + kk);
              b[r] = *reinterpret_cast<const float4*>(hrow[r] + kk + 4);
            }
          }
        }
      };
#pragma unroll
      for (int d = 0; d < PF; ++d) fetch(d, ha[d], hb[d], ga[d], gb[d]);
      bool pok = true;
      for (int i0 = 0; i0 < n_kb && pok; i0 += PF) {
#pragma unroll
        for (int d = 0; d < PF; ++d) {
          const int i = i0 + d;
          if (i >= n_kb || !pok) break;
          const int s = i % C::STAGES;
          const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
          if (i >= C::STAGES) {
            int w_ok = 1;
            if (lane == 0 && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag)) {
              abort_flag = 1; record_failure(p.err, 4); w_ok = 0;
            }
            pok = __shfl_sync(0xffffffffu, w_ok, 0) != 0;
            if (!pok) break;
          }
          uint8_t* bt = smem + (size_t)s * C::STAGE_BYTES + W_BYTES;
          float gv[8];
          if (p.norm.g_is_bf16) {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&ga[d]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { gv[2 * e] = __low2float(h2[e]); gv[2 * e + 1] = __high2float(h2[e]); }
          } else {
            gv[0] = __uint_as_float(ga[d].x); gv[1] = __uint_as_float(ga[d].y);
            gv[2] = __uint_as_float(ga[d].z); gv[3] = __uint_as_float(ga[d].w);
            gv[4] = __uint_as_float(gb[d].x); gv[5] = __uint_as_float(gb[d].y);
            gv[6] = __uint_as_float(gb[d].z); gv[7] = __uint_as_float(gb[d].w);
          }
#pragma unroll
          for (int r = 0; r < RPT; ++r) {
            const int t = (pt >> 3) + 16 * r;
            const float4 a = ha[d][r], b = hb[d][r];     // zeros outside the matrix
            float acc = ss[r];
            acc = fmaf(a.x, a.x, acc); acc = fmaf(a.y, a.y, acc); acc = fmaf(a.z, a.z, acc); acc = fmaf(a.w, a.w, acc);
            acc = fmaf(b.x, b.x, acc); acc = fmaf(b.y, b.y, acc); acc = fmaf(b.z, b.z, acc); acc = fmaf(b.w, b.w, acc);
            ss[r] = acc;
            uint4 o;
            o.x = pack_bf16x2(a.x * gv[0], a.y * gv[1]); o.y = pack_bf16x2(a.z * gv[2], a.w * gv[3]);
            o.z = pack_bf16x2(b.x * gv[4], b.y * gv[5]); o.w = pack_bf16x2(b.z * gv[6], b.w * gv[7]);
            *reinterpret_cast<uint4*>(bt + t * 128 + ((j ^ (t & 7)) << 4)) = o;
          }
          fetch(i + PF, ha[d], hb[d], ga[d], gb[d]);       // the stage PF ahead takes these registers
          fence_proxy_async();                            // generic-proxy stores -> visible to the MMA's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[s]);
        }
      }
      // the eight threads of a token row hold its parts: a fixed tree, then one of them parks the sum
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        float v = ss[r];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (j == 0) ss_part[(pt >> 3) + 16 * r] = v;
      }
      epilogue_warps_sync();
    }
    bool ok = mbar_wait(&acc_bar, 0, &abort_flag);
    if (!ok) { abort_flag = 1; record_failure(p.err, 3); }
    ok = __all_sync(0xffffffffu, ok);
    epi_ok = ok;
    tc_fence_after();
    const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    if (ok && !landing) {
      // ---- one CTA holds the whole sum: straight from TMEM to the output
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (t0 + c0 >= p.T) break;
        uint32_t g[16], u[16];
        ld_acc(taddr + c0, g);
        if (DUAL) ld_acc(taddr + BN + c0, u);
        tmem_ld_wait();
        if (NORM) {
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) {
            const float rs = rsqrtf(ss_part[c0 + jj] * inv_k + p.norm.eps);
            g[jj] = __float_as_uint(__uint_as_float(g[jj]) * rs);
            if (DUAL) u[jj] = __float_as_uint(__uint_as_float(u[jj]) * rs);
          }
        }
        if (n < p.N) {
          if (EPI == EPI_ACCUM_F32) {
            // all sixteen residual values are fetched before the first store, so the loads overlap
            float* cp = (float*)p.C + (size_t)(t0 + c0) * p.ldc + n;
            float r[16];
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) r[jj] = (t0 + c0 + jj < p.T) ? __ldcg(cp + (size_t)jj * p.ldc) : 0.f;
#pragma unroll
            for (int jj = 0; jj < 16; ++jj)
              if (t0 + c0 + jj < p.T) cp[(size_t)jj * p.ldc] = r[jj] + __uint_as_float(g[jj]);
          } else {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              const int t = t0 + c0 + jj;
              if (t < p.T) emit<EPI>(p, t, n, __uint_as_float(g[jj]), DUAL ? __uint_as_float(u[jj]) : 0.f);
            }
          }
        }
      }
    }
  }

  if (landing) {
    // ---------------------------------------------------------- the ranks' parts meet at the column's owner
    // Token tiles of 16: column c belongs to rank c % ranks, one float per store. Wider tiles:
    // rank r owns the cpr columns from r * cpr (cpr a multiple of 4, ranks a power of two), a
    // thread's values for four columns travel as one 16-byte store, and the owner reads them
    // back four at a time.
    constexpr bool VEC = C::VEC;
    const int ncols = min(BN, p.T - t0);                      // token columns that exist
    const int cpr = VEC ? (((BN + p.splits - 1) / p.splits + 3) & ~3) : (BN + p.splits - 1) / p.splits;
    __syncwarp();
    tc_fence_before();
    if (clustered) {
      // every landing area may be written: its CTA runs (own area) / its products are done (ring)
      if (!C::DEDICATED) cluster_arrive();
      cluster_wait();
    }
    if (epi_warp && epi_ok) {
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t land_cta = smem_u32(land);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= ncols) break;
        uint32_t g[16], u[16];
        ld_acc(taddr + c0, g);
        if (DUAL) ld_acc(taddr + BN + c0, u);
        tmem_ld_wait();
        if constexpr (VEC) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int c = c0 + 4 * q;
            if (c < ncols) {
              // [rank][accumulator][group of four columns][row] x 16 bytes: the rows of a warp lie side
              // by side, so neither these stores nor the owner's loads meet in a bank
              const int owner = c / cpr, slot = c % cpr;
              const uint32_t off = (uint32_t)(((((rank * ACCS) * (cpr >> 2) + (slot >> 2)) * BM) + row) * 16);
              const uint32_t dst = (clustered ? map_to_rank(land_cta, (uint32_t)owner) : land_cta) + off;
              st_cluster_v4(dst, __uint_as_float(g[4 * q]), __uint_as_float(g[4 * q + 1]),
                            __uint_as_float(g[4 * q + 2]), __uint_as_float(g[4 * q + 3]));
              if (DUAL) st_cluster_v4(dst + (uint32_t)((cpr >> 2) * BM * 16), __uint_as_float(u[4 * q]),
                                      __uint_as_float(u[4 * q + 1]), __uint_as_float(u[4 * q + 2]),
                                      __uint_as_float(u[4 * q + 3]));
            }
          }
        } else {
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) {
            const int c = c0 + jj;
            if (c < ncols) {
              const int owner = c % p.splits, slot = c / p.splits;
              const uint32_t off = (uint32_t)((((rank * cpr + slot) * ACCS) * BM + row) * 4);
              if (clustered) {
                const uint32_t dst = map_to_rank(land_cta, (uint32_t)owner) + off;
                st_cluster_f32(dst, __uint_as_float(g[jj]));
                if (DUAL) st_cluster_f32(dst + BM * 4, __uint_as_float(u[jj]));
              } else {
                land[off / 4] = __uint_as_float(g[jj]);
                if (DUAL) land[off / 4 + BM] = __uint_as_float(u[jj]);
              }
            }
          }
        }
      }
      if (NORM && row < ncols) {
        const int owner = VEC ? row / cpr : row % p.splits, slot = VEC ? row % cpr : row / p.splits;
        if (clustered) st_cluster_f32(map_to_rank(smem_u32(&ss_land[rank * BN + slot]), (uint32_t)owner), ss_part[row]);
        else ss_land[slot] = ss_part[row];
      }
    }
    __syncwarp();
    if (clustered) { cluster_arrive(); cluster_wait(); } else __syncthreads();     // every part has landed
    if (epi_warp && !abort_flag) {
      // the pair partner of this row under the rotary epilogue (same tile: heads do not straddle tiles)
      int prow = row;
      if (ROPE) {
        const int d = n % p.rope.hd, half = p.rope.rot_dim >> 1;
        if (d < p.rope.rot_dim) prow = d < half ? row + half : row - half;
      }
      if constexpr (VEC) {
#pragma unroll 1
        for (int slot = 0; slot < cpr && rank * cpr + slot < ncols; slot += 4) {
          const int c = rank * cpr + slot;                     // first of four columns owned here
          float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
          float ssum[4] = {0.f, 0.f, 0.f, 0.f};
          if (EPI == EPI_ACCUM_F32 && n < p.N) {               // the four residual values, loads in flight together
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (c + e < ncols) g[e] = __ldcg((const float*)p.C + (size_t)(t0 + c + e) * p.ldc + n);
          }
#pragma unroll
          for (int s = 0; s < MAX_CLUSTER; ++s) {              // rank order
            if (s < p.splits) {
              const float4* base = reinterpret_cast<const float4*>(land) + (size_t)((s * ACCS) * (cpr >> 2) + (slot >> 2)) * BM;
              const float4 vg = base[row];
              g[0] += vg.x; g[1] += vg.y; g[2] += vg.z; g[3] += vg.w;
              if (DUAL) {
                const float4 vu = base[(size_t)(cpr >> 2) * BM + row];
                u[0] += vu.x; u[1] += vu.y; u[2] += vu.z; u[3] += vu.w;
              }
              if (ROPE) {
                const float4 vw = base[prow];
                w[0] += vw.x; w[1] += vw.y; w[2] += vw.z; w[3] += vw.w;
              }
              if (NORM) {
                const float4 vs = *reinterpret_cast<const float4*>(&ss_land[s * BN + slot]);
                ssum[0] += vs.x; ssum[1] += vs.y; ssum[2] += vs.z; ssum[3] += vs.w;
              }
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int t = t0 + c + e;
            if (c + e >= ncols || n >= p.N) continue;
            float ge = g[e], ue = u[e], we = w[e];
            if (NORM) {
              const float rs = rsqrtf(ssum[e] * inv_k + p.norm.eps);
              ge *= rs; ue *= rs; we *= rs;
            }
            if (ROPE) emit_rope(p, t, n, ge, we);
            else if (EPI == EPI_ACCUM_F32) ((float*)p.C)[(size_t)t * p.ldc + n] = ge;   // residual + ranks in order
            else emit<EPI>(p, t, n, ge, ue);
          }
        }
      } else {
#pragma unroll 1
        for (int slot = 0; slot * p.splits + rank < ncols; ++slot) {
          const int t = t0 + slot * p.splits + rank;
          float g = 0.f, u = 0.f, w = 0.f, ssum = 0.f;
          if (EPI == EPI_ACCUM_F32 && n < p.N) g = __ldcg((const float*)p.C + (size_t)t * p.ldc + n);   // residual
          float pg[MAX_CLUSTER], pu[MAX_CLUSTER], pw[MAX_CLUSTER], ps[MAX_CLUSTER];
#pragma unroll
          for (int s = 0; s < MAX_CLUSTER; ++s) {
            pg[s] = pu[s] = pw[s] = ps[s] = 0.f;
            if (s < p.splits) {
              const float* base = land + (size_t)((s * cpr + slot) * ACCS) * BM;
              pg[s] = base[row];
              if (DUAL) pu[s] = base[BM + row];
              if (ROPE) pw[s] = base[prow];
              if (NORM) ps[s] = ss_land[s * BN + slot];
            }
          }
#pragma unroll
          for (int s = 0; s < MAX_CLUSTER; ++s) { g += pg[s]; u += pu[s]; w += pw[s]; ssum += ps[s]; }   // rank order
          if (NORM) {
            const float rs = rsqrtf(ssum * inv_k + p.norm.eps);
            g *= rs; u *= rs; w *= rs;
          }
          if (n < p.N) {
            if (ROPE) emit_rope(p, t, n, g, w);
            else if (EPI == EPI_ACCUM_F32) ((float*)p.C)[(size_t)t * p.ldc + n] = g;   // residual + ranks in order
            else emit<EPI>(p, t, n, g, u);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// ---------------------------------------------------------------------------- many tokens
// The same product for steps of more than 64 tokens (prompt portions). One CTA per SM walks the
// output tiles (token tiles fastest, so the CTAs of a wave share their weight tiles in L2 and a
// weight byte comes from DRAM once) and keeps two accumulators in TMEM: while the epilogue warps
// read tile i out of one, the MMA warp already fills the other with tile i + 1, so the tensor
// cores do not wait for the epilogue. No ranges of K and no norm in front here; the rotary epilogue
// exists but is chosen only up to 128 tokens (beyond, the row-parallel rotation kernel is faster
// than rotating in four epilogue warps).
// WR: weight rows of a tile per accumulator. 128, or 64 for the kernel with the tokens on the accumulator's
// rows when the 128-row tiles would leave most SMs without one (few tokens).
template <int BN, bool DUAL, int WR = BM> struct PCfg {
  static constexpr int A_TILES = DUAL ? 2 : 1;
  static constexpr int A_BYTES = WR * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int W_BYTES = A_TILES * A_BYTES;
  static constexpr int STAGE_BYTES = W_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = 208 * 1024 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES;
  static constexpr int ACC_COLS = WR == BM ? A_TILES * BN : A_TILES * WR;   // one accumulator set (WR < 128: tokens on the rows)
  static constexpr int TMEM_COLS = 2 * ACC_COLS <= 64 ? 64 : 2 * ACC_COLS <= 128 ? 128 : 2 * ACC_COLS <= 256 ? 256 : 512;
  static_assert(2 * ACC_COLS <= 512, "two accumulator sets must fit in TMEM");
};

template <int BN, int EPI, bool SWAP, int WR = BM>
__global__ void __launch_bounds__(THREADS_MANY, 1)
tc_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                          const Params p) {
  constexpr bool DUAL = (EPI == EPI_SWIGLU);
  constexpr bool ROPE = (EPI == EPI_QKV_ROPE);
  static_assert(!SWAP || (DUAL && BN == 128), "tokens on the accumulator's rows: gate/up pairs, 128 tokens x 128 or 64 features a tile");
  static_assert(WR == BM || (SWAP && WR == 64), "tiles of 64 weight rows only with the tokens on the accumulator's rows");
  typedef PCfg<BN, DUAL, WR> C;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];      // MMA warp -> epilogue: this accumulator set is complete
  __shared__ __align__(8) uint64_t acc_empty[2];     // epilogue -> MMA warp: it has been read out
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int never_flag;
  // rotary epilogue: a row's pair partner lies 16+ rows away, in another warp's TMEM lanes; the
  // epilogue warps pass 32 columns at a time through this buffer
  constexpr int XS = BM + 4;
  __shared__ __align__(16) float xch[ROPE ? 32 * XS : 4];
  __shared__ long long tok_off[ROPE ? BN : 1];
  __shared__ int epi_fail;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int bn = p.bn;                                   // tokens per tile: chosen by the host so that the tiles fill whole waves
  const int t_tiles = (p.T + bn - 1) / bn, n_tiles = (p.N + WR - 1) / WR;
  const int tiles = t_tiles * n_tiles;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    abort_flag = 0;
    never_flag = 0;
    epi_fail = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_w); prefetch_tensormap(&tmap_x); }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_x = policy_evict_last();    // the token tiles are read by every weight tile
      pdl_wait();                                    // activations come from the kernel before
      int it = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int t0 = (tile % t_tiles) * bn, n0 = (tile / t_tiles) * WR;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
          if (it >= C::STAGES && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag)) {
            abort_flag = 1; record_failure(p.err, 5); ok = false; break;
          }
          uint8_t* st = smem + (size_t)s * C::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], (uint32_t)(C::W_BYTES + bn * BK * 2));
          const int k = kb * BK;
          tma_load_2d(st, &tmap_w, &full_bar[s], k, n0);
          if (DUAL) tma_load_2d(st + C::A_BYTES, &tmap_w, &full_bar[s], k, p.up_row0 + n0);
          tma_load_2d_hint(st + C::W_BYTES, &tmap_x, &full_bar[s], k, t0, pol_x);
          issued = it + 1;
        }
      }
      if (abort_flag) {
        for (int i = max(0, issued - C::STAGES); i < issued; ++i)
          mbar_wait(&full_bar[i % C::STAGES], (uint32_t)(i / C::STAGES) & 1u, &never_flag, 200000000LL);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // SWAP: the 128 tokens are the rows and the tile's 128 (64) gate and 128 (64) up weight rows, which
      // lie one after the other in a stage, the 256 (128) columns of one product
      const uint32_t idesc = SWAP ? umma_idesc_bf16(BM, 2 * WR) : umma_idesc_bf16(BM, bn);
      int it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++ti) {
        const int buf = ti & 1, use = ti >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (uint32_t)(use - 1) & 1u, &abort_flag)) {
          abort_flag = 1; record_failure(p.err, 6); ok = false; break;
        }
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + (uint32_t)(buf * C::ACC_COLS);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, &abort_flag)) { abort_flag = 1; record_failure(p.err, 2); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::W_BYTES;
          const uint64_t da = umma_desc_sw128(a_addr);
          const uint64_t db = umma_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            const uint64_t koff = (uint64_t)(k * UMMA_K * 2 / 16);
            if (SWAP) { umma_bf16(acc_addr, db + koff, da + koff, idesc, acc); continue; }
            umma_bf16(acc_addr, da + koff, db + koff, idesc, acc);
            if (DUAL) {
              const uint64_t du = umma_desc_sw128(a_addr + C::A_BYTES);
              umma_bf16(acc_addr + BN, du + koff, db + koff, idesc, acc);
            }
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..9): a warp reads the
    // TMEM lanes of its quarter (warp % 4); the two warps of a quarter take half of the token columns
    // each. One warp on a scheduler waits out every instruction's latency alone, so an epilogue's time
    // goes with the instructions per warp, and the last tile's epilogue is not hidden by a mainloop.
    const int row = (warp & 3) * 32 + lane;
    const int grp = (warp - 2) >> 2;
    pdl_wait();
    int ti = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++ti) {
      const int t0 = (tile % t_tiles) * bn, n0 = (tile / t_tiles) * WR;
      const int n = n0 + row;
      const int buf = ti & 1, use = ti >> 1;
      ok = mbar_wait(&acc_full[buf], (uint32_t)use & 1u, &abort_flag);
      if (!ok) { abort_flag = 1; record_failure(p.err, 3); }
      ok = __all_sync(0xffffffffu, ok);
      if (ROPE) {                                        // the eight warps leave together or not at all
        if (!ok) epi_fail = 1;
        epilogue8_sync();
        ok = epi_fail == 0;
      }
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * C::ACC_COLS);
      if (SWAP) {
        // this thread's row is a token; its gate values are columns 0..WR-1, its up values WR..2 WR-1. The
        // first warp of a quarter takes the lower half of the features, the second the upper, 32 at a
        // time, and writes them as 16-byte pieces of the token's output row.
        const int t = t0 + row;
        bf16* crow = (bf16*)p.C + (size_t)t * p.ldc + n0;
#pragma unroll 1
        for (int c0 = grp * (WR / 2); c0 < grp * (WR / 2) + WR / 2; c0 += 32) {
          if (n0 + c0 >= p.N) break;
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c0, g);
          tmem_ld32(taddr + WR + c0, u);
          tmem_ld_wait();
          if (t < p.T) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (n0 + c0 + 8 * q >= p.N) break;
              float h[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float gv = __uint_as_float(g[8 * q + e]);
                h[e] = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[8 * q + e]);   // float, rounded once to bfloat16
              }
              uint4 pk;
              pk.x = pack_bf16x2(h[0], h[1]); pk.y = pack_bf16x2(h[2], h[3]);
              pk.z = pack_bf16x2(h[4], h[5]); pk.w = pack_bf16x2(h[6], h[7]);
              *reinterpret_cast<uint4*>(crow + c0 + 8 * q) = pk;
            }
          }
        }
      } else if (ROPE) {
        // Rotation needs a row's pair partner, which lies half a head away in another warp's TMEM lanes, and
        // with one warp on each scheduler an epilogue is bound by the instructions it issues. So 32 token
        // columns at a time go through shared memory ([token][row], rows padded by 4 against bank
        // conflicts), and from there each of the 256 threads takes, for one token, two groups of 8
        // neighbouring rows: values, partners and angles as 16-byte loads, the rotated result as one
        // 16-byte store into C and one into the cache.
        // (a row's place in the buffer has bit 2 flipped in the upper half of each 64 rows, so that the
        // eight threads of a 16-byte read, 8 rows apart, meet 32 different banks)
        auto xrow = [](int r_) { return r_ ^ (((r_ >> 5) & 1) << 2); };
        const RopeArgs& r = p.rope;
        const int et = (warp - 2) * 32 + lane, tt = et >> 3, q8 = (et & 7) * 8;
        const int half = r.rot_dim >> 1;
        bool g_turn[2], g_low[2], g_live[2];
        int g_fi[2], g_part[2];
        bf16* g_cache[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int rb = q8 + 64 * k, nn = n0 + rb;
          const int head = nn / r.hd, d = nn - head * r.hd;
          g_live[k] = nn < p.N;
          g_turn[k] = g_live[k] && head < r.nh + r.nkv && d < r.rot_dim;
          g_low[k] = d < half;
          g_fi[k] = g_low[k] ? d : d - half;
          g_part[k] = g_turn[k] ? (g_low[k] ? rb + half : rb - half) : rb;
          const bool is_k = head < r.nh + r.nkv;
          g_cache[k] = (g_live[k] && head >= r.nh && r.slots != nullptr)
              ? (is_k ? r.kcache : r.vcache) + (size_t)(head - r.nh - (is_k ? 0 : r.nkv)) * r.page_size * r.hd + d : nullptr;
        }
        // where each token of the tile starts in a cache (elements; -1: not written), once for all rows
        if (r.slots != nullptr) {
          for (int c = et; c < bn; c += 256) {
            const int t = t0 + c;
            const int slot = t < p.T ? r.slots[t] : -1;
            tok_off[c] = slot >= 0 ? ((long long)(slot / r.page_size) * r.nkv * r.page_size + slot % r.page_size) * r.hd : -1ll;
          }
        }
        // This thread's angles are asked for one chunk ahead, all at once: they come from L2, which is
        // busy with the operands, and a chunk that waited for its own would wait about as long again
        // as it works.
        float4 ang[2][4], ang_next[2][4];
        auto ask_angles = [&](int c0, float4 (&a)[2][4]) {
          if (r.cos_sin == nullptr || t0 + c0 >= p.T) return;
          const float2* trow = r.cos_sin + (size_t)min(t0 + c0 + tt, p.T - 1) * half;
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (g_turn[k]) {
#pragma unroll
              for (int i = 0; i < 4; ++i) a[k][i] = __ldg(reinterpret_cast<const float4*>(trow + g_fi[k]) + i);
            }
          }
        };
        ask_angles(0, ang_next);
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 32) {
          if (t0 + c0 >= p.T) break;
#pragma unroll
          for (int k = 0; k < 2; ++k)
#pragma unroll
            for (int i = 0; i < 4; ++i) ang[k][i] = ang_next[k][i];
          if (c0 + 32 < bn) ask_angles(c0 + 32, ang_next);
          {
            uint32_t g[16];                               // 16 of the 32 columns from each warp of a quarter
            tmem_ld16(taddr + c0 + 16 * grp, g);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) xch[(16 * grp + jj) * XS + xrow(row)] = __uint_as_float(g[jj]);
          }
          epilogue8_sync();
          const int t = t0 + c0 + tt;
          if (t < p.T && c0 + tt < bn) {
            const float* xr = xch + tt * XS;
            const long long coff = r.slots != nullptr ? tok_off[c0 + tt] : -1ll;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              if (!g_live[k]) continue;
              const float4 v0 = *reinterpret_cast<const float4*>(xr + xrow(q8 + 64 * k));
              const float4 v1 = *reinterpret_cast<const float4*>(xr + xrow(q8 + 64 * k + 4));
              float o[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
              if (g_turn[k]) {
                const float4 w0 = *reinterpret_cast<const float4*>(xr + xrow(g_part[k]));
                const float4 w1 = *reinterpret_cast<const float4*>(xr + xrow(g_part[k] + 4));
                const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                float cs[8], sn[8];
                if (r.cos_sin != nullptr) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float4 a = ang[k][i];
                    cs[2 * i] = a.x; sn[2 * i] = a.y; cs[2 * i + 1] = a.z; sn[2 * i + 1] = a.w;
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 8; ++i) { const float2 a = angle_of(r, t, g_fi[k] + i); cs[i] = a.x; sn[i] = a.y; }   // no table given
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = g_low[k] ? o[i] * cs[i] - w[i] * sn[i] : w[i] * sn[i] + o[i] * cs[i];
              }
              uint4 pk;
              pk.x = pack_bf16x2(o[0], o[1]); pk.y = pack_bf16x2(o[2], o[3]);
              pk.z = pack_bf16x2(o[4], o[5]); pk.w = pack_bf16x2(o[6], o[7]);
              *reinterpret_cast<uint4*>((bf16*)p.C + (size_t)t * p.ldc + n0 + q8 + 64 * k) = pk;
              if (g_cache[k] != nullptr && coff >= 0) *reinterpret_cast<uint4*>(g_cache[k] + coff) = pk;
            }
          }
          epilogue8_sync();                               // all have read before the next 32 columns come in
        }
      } else {
        // The tile leaves TMEM 64 token columns at a time (32 of each half of a gate/up pair): a load from
        // TMEM and the wait for it are a round trip of their own, and sixteen of them for a tile of 256
        // columns were most of what the epilogue took. The residual values of the same columns are
        // fetched while the accumulator values are on their way.
        // (with ten warps a thread has 168 registers: the residual's 64 beside the accumulator's 64 would spill)
        constexpr int CW = (DUAL || BN < 128 || EPI == EPI_ACCUM_F32) ? 32 : 64;
        float* cbase = (float*)p.C + (size_t)t0 * p.ldc + n;
        // the first warp of a quarter takes the columns up to `mid` (a multiple of 32), the second the rest;
        // `lim`: columns of this warp that are tokens of the tile and of the step
        const int mid = ((bn / 2 + 31) / 32) * 32;
        const int c_begin = grp == 0 ? 0 : mid;
        const int lim = min(grp == 0 ? mid : bn, p.T - t0);
#pragma unroll 1
        for (int c0 = c_begin; c0 < lim; c0 += CW) {
          uint32_t g[CW], u[DUAL ? CW : 1];
          float r[EPI == EPI_ACCUM_F32 ? CW : 1];
          if (DUAL) {
            tmem_ld32(taddr + c0, reinterpret_cast<uint32_t(&)[32]>(g));
            tmem_ld32(taddr + BN + c0, reinterpret_cast<uint32_t(&)[32]>(u));
          } else if (CW == 32) {
            tmem_ld32(taddr + c0, reinterpret_cast<uint32_t(&)[32]>(g));
          } else {
            tmem_ld64(taddr + c0, reinterpret_cast<uint32_t(&)[64]>(g));
          }
          if (EPI == EPI_ACCUM_F32 && n < p.N) {
            const float* cp = cbase + (size_t)c0 * p.ldc;
#pragma unroll
            for (int jj = 0; jj < CW; ++jj) r[jj] = (c0 + jj < lim) ? __ldcg(cp + (size_t)jj * p.ldc) : 0.f;
          }
          tmem_ld_wait();
          if (n < p.N) {
            if (EPI == EPI_ACCUM_F32) {
              float* cp = cbase + (size_t)c0 * p.ldc;
#pragma unroll
              for (int jj = 0; jj < CW; ++jj)
                if (c0 + jj < lim) cp[(size_t)jj * p.ldc] = r[jj] + __uint_as_float(g[jj]);
            } else if (EPI == EPI_STORE) {
              bf16* cp = (bf16*)p.C + (size_t)(t0 + c0) * p.ldc + n;
#pragma unroll
              for (int jj = 0; jj < CW; ++jj, cp += p.ldc)
                if (c0 + jj < lim) *cp = __float2bfloat16_rn(__uint_as_float(g[jj]));
            } else {
#pragma unroll
              for (int jj = 0; jj < CW; ++jj) {
                if (c0 + jj < lim) emit<EPI>(p, t0 + c0 + jj, n, __uint_as_float(g[jj]), DUAL ? __uint_as_float(u[jj]) : 0.f);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);      // this warp's quarter of the set is read out
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// ---------------------------------------------------------------------------- many tokens, two SMs a tile
// The same persistent scheme on pairs of CTAs (a cluster of two, `tcgen05.mma.cta_group::2`): a tile is
// 256 weight rows x BN tokens; each CTA of the pair loads its own 128 weight rows and its own half of
// the token tile into its own shared memory (plain TMA loads, no multicast) and keeps its 128
// accumulator rows in its own TMEM; the even CTA issues the MMAs, which read both CTAs' shared
// memory. Per FLOP an SM takes in a third fewer operand bytes than alone (32 KB instead of 48 KB per
// 64 of K at BN = 256), and operand bytes into the SM are what bounds the one-SM kernel above.
// Hand-overs: a stage's bytes from both CTAs are counted by the even CTA's `full` barrier (the odd
// CTA's loads name it by its cluster address); the even CTA's MMA thread commits to both CTAs' `empty`
// and `acc_full` barriers; both CTAs' epilogue warps arrive at the even CTA's `acc_empty`. Both CTAs
// allocate and free TMEM, and meet at a cluster barrier before they free it and leave, so that no
// signal or MMA ever addresses a CTA that is gone. Every wait is bounded.
template <int BN, bool DUAL> struct PairCfg {
  static constexpr int A_TILES = DUAL ? 2 : 1;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;              // this CTA's half of the token tile
  static constexpr int W_BYTES = A_TILES * A_BYTES;
  static constexpr int STAGE_BYTES = W_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = 208 * 1024 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES;
  static constexpr int ACC_COLS = A_TILES * BN;
  static constexpr int TMEM_COLS = 2 * ACC_COLS <= 64 ? 64 : 2 * ACC_COLS <= 128 ? 128 : 2 * ACC_COLS <= 256 ? 256 : 512;
  static_assert(2 * ACC_COLS <= 512, "two accumulator sets must fit in TMEM");
};
constexpr long long PAIR_WAIT_CYCLES = 1000000000LL;             // about half a second

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const Params p) {
  constexpr bool DUAL = (EPI == EPI_SWIGLU);
  typedef PairCfg<BN, DUAL> C;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::STAGES];     // used in the even CTA: both CTAs' bytes of a stage
  __shared__ __align__(8) uint64_t empty_bar[C::STAGES];    // in each CTA: the pair's MMAs have read the stage
  __shared__ __align__(8) uint64_t acc_full[2];             // in each CTA: the accumulator set is complete
  __shared__ __align__(8) uint64_t acc_empty[2];            // used in the even CTA: both CTAs have read the set out
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int never_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int t_tiles = (p.T + BN - 1) / BN, n_tiles = (p.N + 2 * BM - 1) / (2 * BM);
  const int tiles = t_tiles * n_tiles;
  const int n_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    abort_flag = 0;
    never_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmap_w); prefetch_tensormap(&tmap_x); }
  if (warp == 1) { tmem_alloc_pair(&tmem_base_slot, C::TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();          // the peer's barriers exist before anything is signalled there
  pdl_launch();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (in both CTAs)
    if (lane == 0) {
      pdl_wait();
      int it = 0, issued = 0;
      bool ok = true;
      for (int tile = pair_id; tile < tiles && ok; tile += n_pairs) {
        const int t0 = (tile % t_tiles) * BN + (int)rank * (BN / 2);
        const int n0 = (tile / t_tiles) * (2 * BM) + (int)rank * BM;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
          if (it >= C::STAGES && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag, PAIR_WAIT_CYCLES)) {
            abort_flag = 1; record_failure(p.err, 5, (int)rank); ok = false; break;
          }
          uint8_t* st = smem + (size_t)s * C::STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
          const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);
          const int k = kb * BK;
          tma_load_2d_pair(st, &tmap_w, bar, k, n0);
          if (DUAL) tma_load_2d_pair(st + C::A_BYTES, &tmap_w, bar, k, p.up_row0 + n0);
          tma_load_2d_pair(st + C::W_BYTES, &tmap_x, bar, k, t0);
          issued = it + 1;
        }
      }
      (void)issued;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN);
      int it = 0, ti = 0;
      bool ok = true;
      for (int tile = pair_id; tile < tiles && ok; tile += n_pairs, ++ti) {
        const int buf = ti & 1, use = ti >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (uint32_t)(use - 1) & 1u, &abort_flag, PAIR_WAIT_CYCLES)) {
          abort_flag = 1; record_failure(p.err, 6); ok = false; break;
        }
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + (uint32_t)(buf * C::ACC_COLS);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, &abort_flag, PAIR_WAIT_CYCLES)) { abort_flag = 1; record_failure(p.err, 2); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(a_addr);
          const uint64_t db = umma_desc_sw128(a_addr + C::W_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            const uint64_t koff = (uint64_t)(k * UMMA_K * 2 / 16);
            umma_bf16_pair(acc_addr, da + koff, db + koff, idesc, acc);
            if (DUAL) umma_bf16_pair(acc_addr + BN, umma_desc_sw128(a_addr + C::A_BYTES) + koff, db + koff, idesc, acc);
          }
          umma_commit_pair_both(&empty_bar[s]);      // the stage is free, in both CTAs
        }
        if (ok) {
          umma_commit_pair_both(&acc_full[buf]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5), in both CTAs
    const int row = (warp & 3) * 32 + lane;
    const uint32_t drained = map_to_rank(smem_u32(&acc_empty[0]), 0);        // the even CTA's acc_empty[0]
    pdl_wait();
    int ti = 0;
    bool ok = true;
    for (int tile = pair_id; tile < tiles && ok; tile += n_pairs, ++ti) {
      const int t0 = (tile % t_tiles) * BN, n0 = (tile / t_tiles) * (2 * BM) + (int)rank * BM;
      const int n = n0 + row;
      const int buf = ti & 1, use = ti >> 1;
      ok = mbar_wait(&acc_full[buf], (uint32_t)use & 1u, &abort_flag, PAIR_WAIT_CYCLES);
      if (!ok) { abort_flag = 1; record_failure(p.err, 3, (int)rank); }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * C::ACC_COLS);
      // 64 token columns at a time, the residual values fetched while the accumulator's are on their way
      // (as in tc_gemm_persistent_kernel)
      constexpr int CW = DUAL ? 32 : 64;
      float* cbase = (float*)p.C + (size_t)t0 * p.ldc + n;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CW) {
        if (t0 + c0 >= p.T) break;
        uint32_t g[CW], u[DUAL ? CW : 1];
        float r[EPI == EPI_ACCUM_F32 ? CW : 1];
        if (DUAL) {
          tmem_ld32(taddr + c0, reinterpret_cast<uint32_t(&)[32]>(g));
          tmem_ld32(taddr + BN + c0, reinterpret_cast<uint32_t(&)[32]>(u));
        } else {
          tmem_ld64(taddr + c0, reinterpret_cast<uint32_t(&)[64]>(g));
        }
        if (EPI == EPI_ACCUM_F32 && n < p.N) {
          const float* cp = cbase + (size_t)c0 * p.ldc;
#pragma unroll
          for (int jj = 0; jj < CW; ++jj) r[jj] = (t0 + c0 + jj < p.T) ? __ldcg(cp + (size_t)jj * p.ldc) : 0.f;
        }
        tmem_ld_wait();
        if (n < p.N) {
          if (EPI == EPI_ACCUM_F32) {
            float* cp = cbase + (size_t)c0 * p.ldc;
#pragma unroll
            for (int jj = 0; jj < CW; ++jj)
              if (t0 + c0 + jj < p.T) cp[(size_t)jj * p.ldc] = r[jj] + __uint_as_float(g[jj]);
          } else {
#pragma unroll
            for (int jj = 0; jj < CW; ++jj) {
              const int t = t0 + c0 + jj;
              if (t < p.T) emit<EPI>(p, t, n, __uint_as_float(g[jj]), DUAL ? __uint_as_float(u[jj]) : 0.f);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(drained + (uint32_t)(buf * 8));   // this warp's quarter of this CTA's half is read out
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs are done with each other's shared memory, barriers and TMEM
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, C::TMEM_COLS); }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;

int get_encoder() {
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return -5;
  }
  g_encode = (EncodeTiledFn)fn;
  return 0;
}

// bf16 matrix [rows, cols] with row stride ld (elements); box = 64 columns x box_rows rows
int make_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -5;
}

struct MapKey {
  const void* p; long long rows, cols, ld; int box;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows * 1315423911LL + k.cols * 2654435761LL + k.ld) << 1) ^ k.box;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;   // weight maps live as long as the process

int cached_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box) {
  std::lock_guard<std::mutex> lk(g_mu);
  MapKey key{ptr, rows, cols, ld, box};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    int rc = make_map(&m, ptr, rows, cols, ld, box);
    if (rc) return rc;
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

template <int BN, int EPI, bool NORM>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t s) {
  typedef Cfg<BN, EPI == EPI_SWIGLU> C;
  static bool configured[64] = {};
  if (allow_dynamic_smem(tc_gemm_kernel<BN, EPI, NORM>, C::SMEM_BYTES, configured)) return -5;
  return launch_ex(tc_gemm_kernel<BN, EPI, NORM>, grid, dim3(THREADS_SMALL), C::SMEM_BYTES, s, p.splits, mw, mx, p);
}

template <int BN, int EPI, bool SWAP = false, int WR = BM>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int sm_count, cudaStream_t s) {
  typedef PCfg<BN, EPI == EPI_SWIGLU, WR> C;
  static bool configured[64] = {};
  if (allow_dynamic_smem(tc_gemm_persistent_kernel<BN, EPI, SWAP, WR>, C::SMEM_BYTES, configured)) return -5;
  if (p.bn < 16 || p.bn > BN || p.bn % 16) return ERR_BAD_SIZE;
  const int tiles = ((p.T + p.bn - 1) / p.bn) * ((p.N + WR - 1) / WR);
  const int ctas = tiles < sm_count ? tiles : sm_count;
  return launch_ex(tc_gemm_persistent_kernel<BN, EPI, SWAP, WR>, dim3(ctas), dim3(THREADS_MANY), C::SMEM_BYTES, s, 1, mw, mx, p);
}

template <int BN, int EPI>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int sm_count, cudaStream_t s) {
  typedef PairCfg<BN, EPI == EPI_SWIGLU> C;
  static bool configured[64] = {};
  if (allow_dynamic_smem(tc_gemm_pair_kernel<BN, EPI>, C::SMEM_BYTES, configured)) return -5;
  const int tiles = ((p.T + BN - 1) / BN) * ((p.N + 2 * BM - 1) / (2 * BM));
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  // the two CTAs of a pair are neighbours along x: blocks 2i and 2i + 1
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  attrs[n].id = cudaLaunchAttributeClusterDimension;
  attrs[n].val.clusterDim.x = 2; attrs[n].val.clusterDim.y = 1; attrs[n].val.clusterDim.z = 1;
  ++n;
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, tc_gemm_pair_kernel<BN, EPI>, mw, mx, p);
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  return 0;
}

// Whether pairs of CTAs take the products of long prompt portions (rllm_tc_gemm_set_pairs). Off unless asked
// for: measured on a B200 (2,048 tokens, Llama 3.2 1B shapes) the pair kernel gives the same bits and is
// level with the one-SM kernel on the q/k/v product and 4 to 12 % behind on the others; its MMA thread
// waits for operands 40 to 70 % of the time although an SM takes in a third fewer bytes.
bool g_pairs = false;

template <int EPI>
int launch_many(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int sm_count, cudaStream_t s) {
  // the kernel's shared memory and accumulator sets are laid out for up to 64, 128 or 256 tokens a tile
  if (bn <= 64) return launch_persistent<64, EPI>(mw, mx, p, sm_count, s);
  if (bn <= 128) return launch_persistent<128, EPI>(mw, mx, p, sm_count, s);
  if constexpr (EPI != EPI_SWIGLU) { if (bn <= 256) return launch_persistent<256, EPI>(mw, mx, p, sm_count, s); }
  return ERR_BAD_SIZE;
}

template <int EPI>
int launch_bn(int bn, bool norm, const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid,
              cudaStream_t s) {
  if (norm) {
    if constexpr (EPI != EPI_ACCUM_F32) {
      switch (bn) {
        case 16: return launch<16, EPI, true>(mw, mx, p, grid, s);
        case 32: return launch<32, EPI, true>(mw, mx, p, grid, s);
      }
    }
    return ERR_BAD_SIZE;
  }
  switch (bn) {
    case 16: return launch<16, EPI, false>(mw, mx, p, grid, s);
    case 32: return launch<32, EPI, false>(mw, mx, p, grid, s);
  }
  return ERR_BAD_SIZE;
}

// Whether gate/up products of portions of more than 64 tokens put the tokens on the accumulator's rows
// (rllm_tc_gemm_set_token_rows): a tile is then 128 tokens x (128 gate + 128 up weight rows) and one product
// of 256 columns per 16 of K, where weight rows on the accumulator's rows need two of 128 columns, which
// read as many bytes of shared memory per cycle as it delivers. Same bits; 2,048 tokens, 2 x 8,192 x 2,048:
// 99 us against 110.
bool g_token_rows = true;

void plan(int epi, int T, int N, int K, int sm_count, int allow_split, int* bn_out, int* splits_out,
          bool* few_out = nullptr, bool norm = false) {
  const bool dual = epi == EPI_SWIGLU;
  const int n_tiles = (N + BM - 1) / BM;
  int bn, splits = 1;
  const int kb = (K + BK - 1) / BK;
  if (allow_split && n_tiles * 2 <= sm_count) {
    // One CTA per SM, as far as it goes; with a single token tile (up to 32 tokens) and a single
    // weight tile (84 KB of shared memory a CTA) two per SM. More and shorter ranges win as long as
    // the CTAs are resident together: at 8 ranges of a K of 2,048 a CTA's whole share of the weights
    // (64 KB) is in flight before the previous kernel has ended (QKV at 8 tokens: 6.3 us with 6
    // ranges, 5.9 us with 8). With two token tiles the doubled CTAs cost more than they save
    // (64 tokens: 3 to 5 % of the decode step).
    splits = ((!dual && T <= 32) ? 2 * sm_count : sm_count) / n_tiles;
    if (splits > kb / 2) splits = kb / 2;                     // at least two K blocks per range
    if (splits > MAX_CLUSTER) splits = MAX_CLUSTER;
    if (splits < 1) splits = 1;
    // allow_split > 1 asks for that many ranges where ranges are allowed (the microbenchmark's sweep)
    const int forced = allow_split > 1 ? allow_split : 0;
    if (forced > 0) splits = forced < kb / 2 ? (forced < MAX_CLUSTER ? forced : MAX_CLUSTER) : (kb / 2 > 0 ? kb / 2 : 1);
  }
  // A step of few tokens: token tiles of 16 or 32 (33 to 64 tokens: two tiles of 32 land their
  // parts faster than one of 64, which reads the weights once but has three stages and one issuing
  // thread: at 64 tokens gate/up 20.8 against 19.3 us, down 13.7 against 12.2, O 8.3 against 7.3),
  // and ranges of K until every SM has a CTA. Up to 128 tokens the
  // same holds for a narrow weight that would give the persistent kernel under a quarter of the SMs.
  // (33 to 64 tokens against a weight of many tiles, the output head: one token tile of 64 in the persistent
  // kernel reads the weight once, two tiles of 32 read it twice)
  const bool wide_head = T > 32 && T <= 64 && n_tiles >= 4 * sm_count;
  // (33 to 64 tokens against a gate/up pair: the kernel with the tokens on the accumulator's rows, which has
  // no ranges of K to merge and no norm in front, unless the norm is asked for in the same kernel)
  const bool rows_kernel = dual && g_token_rows && !norm && T > 32;
  const bool few = (T <= 64 && !wide_head && !rows_kernel) || (T <= 128 && splits > 1 && n_tiles * ((T + 63) / 64) * 4 <= sm_count);
  if (few) {
    bn = T <= 16 ? 16 : 32;
    if (bn >= 32) while (splits & (splits - 1)) splits &= splits - 1;     // wider tiles: a power of two
  } else {
    // More tokens: no ranges of K (a partial tile of 128+ columns costs more to merge than it saves), and
    // the persistent kernel, whose tile takes any number of tokens in steps of 16. A CTA's time goes with
    // its tiles x the operand rows a tile takes in per 64 of K (128 or 256 weight rows + the tokens): the
    // width that makes this smallest fills whole waves (2,048 tokens x 24 weight tiles: 176 tokens a tile
    // are 288 tiles, 1.95 waves of 148, where 256 are 192 tiles, 1.3 waves that cost 2); of equals the wider.
    splits = 1;
    const int widest = dual ? 128 : 256;
    const long long w_rows = dual ? 256 : 128;
    long long best = -1;
    bn = widest;
    for (int cand = widest; cand >= 64; cand -= 16) {
      const long long tiles = (long long)n_tiles * ((T + cand - 1) / cand);
      const long long waves = (tiles + sm_count - 1) / sm_count;
      const long long cost = waves * (w_rows + cand);
      if (best < 0 || cost < best) { best = cost; bn = cand; }
    }
    // tokens on the accumulator's rows: 128 a tile, also where fewer tokens leave rows empty (96 tokens:
    // 17.8 us against 19.1 with 96 tokens beside the weight rows)
    if (dual && g_token_rows) bn = 128;
  }
  *bn_out = bn;
  *splits_out = splits;
  if (few_out) *few_out = few;
}

// X null: the fused-norm variants (norm must be given, T <= NORM_MAX_T).
int run(int epi, const void* X, long long ldx, const NormArgs* norm, const void* W, void* Cout, long long ldc,
        int T, int N, int K, int allow_split, int* err, int sm_count, const RopeArgs* rope, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) return ERR_BAD_SIZE;                          // TMA: strides multiple of 16 bytes
  if ((uintptr_t)W & 15) return ERR_BAD_ALIGN;
  if (norm) {
    if (T > NORM_MAX_T || epi == EPI_ACCUM_F32) return ERR_BAD_SIZE;
    if (norm->ldh % 4 || ((uintptr_t)norm->h & 15) || ((uintptr_t)norm->g & 15)) return ERR_BAD_ALIGN;
  } else {
    if (ldx % 8) return ERR_BAD_SIZE;
    if ((uintptr_t)X & 15) return ERR_BAD_ALIGN;
  }
  int rc = get_encoder();
  if (rc) return rc;
  int bn, splits;
  bool few;
  plan(epi, T, N, K, sm_count, allow_split, &bn, &splits, &few, norm != nullptr);
  const bool many = !few;            // the persistent kernel (no ranges of K, no norm in front)
  if (many && norm) return ERR_BAD_SIZE;
  const bool dual = epi == EPI_SWIGLU;
  CUtensorMap mw, mx;
  if ((rc = cached_map(&mw, W, dual ? 2LL * N : N, K, K, BM))) return rc;
  // long portions: a tile of 256 weight rows x bn tokens on a pair of CTAs, each loading half of the token tile
  const bool pair = g_pairs && !norm && epi != EPI_QKV_ROPE && sm_count >= 2 && many && T >= (dual ? 128 : 256);
  if (pair) bn = dual ? 128 : 256;                                   // the pair kernel's tile is fixed
  if (norm) mx = mw;                                                 // not used by the kernel
  else if ((rc = make_map(&mx, X, T, K, ldx, pair ? bn / 2 : bn))) return rc;
  Params p;
  p.C = Cout; p.ldc = (int)ldc; p.T = T; p.N = N; p.K = K; p.up_row0 = N; p.splits = splits; p.err = err; p.bn = bn;
  p.rope = rope ? *rope : RopeArgs{};
  p.norm = norm ? *norm : NormArgs{};
  dim3 grid((T + bn - 1) / bn, (N + BM - 1) / BM, splits);
  if (grid.y > 65535) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  const bool nm = norm != nullptr;
  if (pair) {
    switch (epi) {
      case EPI_STORE: return launch_pair<256, EPI_STORE>(mw, mx, p, sm_count, s);
      case EPI_STORE_F32: return launch_pair<256, EPI_STORE_F32>(mw, mx, p, sm_count, s);
      case EPI_ACCUM_F32: return launch_pair<256, EPI_ACCUM_F32>(mw, mx, p, sm_count, s);
      case EPI_SWIGLU: return launch_pair<128, EPI_SWIGLU>(mw, mx, p, sm_count, s);
    }
  }
  if (many && rope) {
    // the persistent kernel's rotary epilogue moves groups of 8 neighbouring features as 16 bytes
    if (rope->hd % 16 || rope->rot_dim % 16 || ldc % 8) return ERR_BAD_SIZE;
    if (((uintptr_t)Cout | (uintptr_t)rope->kcache | (uintptr_t)rope->vcache | (uintptr_t)rope->cos_sin) & 15) return ERR_BAD_ALIGN;
  }
  if (many && dual && g_token_rows && N % 8 == 0 && ldc % 8 == 0 && !((uintptr_t)Cout & 15)) {
    // tiles of 64 gate and 64 up rows where tiles of 128 would leave half of the SMs without one
    const long long tiles128 = (long long)((T + bn - 1) / bn) * ((N + BM - 1) / BM);
    if (tiles128 * 2 <= sm_count + sm_count / 8) {
      CUtensorMap mw64;
      if ((rc = cached_map(&mw64, W, 2LL * N, K, K, 64))) return rc;
      return launch_persistent<128, EPI_SWIGLU, true, 64>(mw64, mx, p, sm_count, s);
    }
    return launch_persistent<128, EPI_SWIGLU, true>(mw, mx, p, sm_count, s);
  }
  if (many) {
    // many tokens: the persistent kernel with two accumulator sets
    switch (epi) {
      case EPI_STORE: return launch_many<EPI_STORE>(bn, mw, mx, p, sm_count, s);
      case EPI_STORE_F32: return launch_many<EPI_STORE_F32>(bn, mw, mx, p, sm_count, s);
      case EPI_ACCUM_F32: return launch_many<EPI_ACCUM_F32>(bn, mw, mx, p, sm_count, s);
      case EPI_SWIGLU: return launch_many<EPI_SWIGLU>(bn, mw, mx, p, sm_count, s);
      case EPI_QKV_ROPE: return launch_many<EPI_QKV_ROPE>(bn, mw, mx, p, sm_count, s);
    }
  }
  switch (epi) {
    case EPI_STORE: return launch_bn<EPI_STORE>(bn, nm, mw, mx, p, grid, s);
    case EPI_STORE_F32: return launch_bn<EPI_STORE_F32>(bn, nm, mw, mx, p, grid, s);
    case EPI_ACCUM_F32: return launch_bn<EPI_ACCUM_F32>(bn, nm, mw, mx, p, grid, s);
    case EPI_SWIGLU: return launch_bn<EPI_SWIGLU>(bn, nm, mw, mx, p, grid, s);
    case EPI_QKV_ROPE: return launch_bn<EPI_QKV_ROPE>(bn, nm, mw, mx, p, grid, s);
  }
  return ERR_BAD_SIZE;
}

}  // namespace

// Token tile and ranges of K (= CTAs per cluster) the launcher would choose.
RLLM_API int rllm_tc_gemm_plan(int epi, int T, int N, int K, int sm_count, int allow_split, int* bn_out,
                               int* splits_out) {
  plan(epi, T, N, K, sm_count, allow_split, bn_out, splits_out);
  return 0;
}

RLLM_API int rllm_tc_gemm_set_pairs(int on) { g_pairs = on != 0; return 0; }
RLLM_API int rllm_tc_gemm_set_token_rows(int on) { g_token_rows = on != 0; return 0; }

// X: [T, K] bf16, row stride ldx; W: [N, K] bf16 contiguous ([2N, K] for SwiGLU: gate rows then up
// rows); C: [T, N] with row stride ldc, bf16 (store, SwiGLU) or float (store-float, accumulate).
// allow_split 0: one CTA per output tile whatever the size; 1: the launcher's choice of ranges of K;
// n > 1: n ranges where ranges are allowed. Returns 0, or a negative refusal.
RLLM_API int rllm_tc_gemm(int epi, const void* X, long long ldx, const void* W, void* Cout, long long ldc,
                          int T, int N, int K, int allow_split, int* err, int sm_count, void* stream) {
  if (epi < 0 || epi > 3 || !X) return ERR_BAD_SIZE;
  return run(epi, X, ldx, nullptr, W, Cout, ldc, T, N, K, allow_split, err, sm_count, nullptr, stream);
}

// The same product with RMSNorm in front, in one kernel: X[t, :] = h[row(t), :] * rsqrt(mean(h^2) + eps) * g,
// row(t) = rows[t], or t when rows is null. h float [*, K] with row stride ldh (a multiple of 4); g the norm
// weight [K], float (g_dt 0) or bfloat16 (g_dt 1). T at most 64 (rllm_tc_gemm_norm_max_tokens); epilogues
// store, store-float and SwiGLU.
RLLM_API int rllm_tc_gemm_norm(int epi, const float* h, long long ldh, const int* rows, const void* g, int g_dt,
                               float eps, const void* W, void* Cout, long long ldc, int T, int N, int K,
                               int allow_split, int* err, int sm_count, void* stream) {
  if (epi < 0 || epi > 3 || epi == EPI_ACCUM_F32 || !h || !g || (g_dt != DT_F32 && g_dt != DT_BF16)) return ERR_BAD_SIZE;
  NormArgs nm;
  nm.h = h; nm.ldh = ldh; nm.rows = rows; nm.g = g; nm.g_is_bf16 = g_dt == DT_BF16; nm.eps = eps;
  return run(epi, nullptr, 0, &nm, W, Cout, ldc, T, N, K, allow_split, err, sm_count, nullptr, stream);
}
RLLM_API int rllm_tc_gemm_norm_max_tokens() { return NORM_MAX_T; }

// The q/k/v projection with the rotary position encoding and the cache write in its epilogue:
// QKV[T, (nh + 2 nkv) * hd] = X W^T; pair (i, i + rot_dim/2) of every q and k head is rotated by
// positions[t] * inv_freq[i]; rotated k and plain v also go to the paged cache at slots[t]
// (slots null or < 0: no write). Head size must divide 128 so that no head straddles two tiles.
// cos_sin: the step's table [T][rot_dim / 2] of (cos, sin), or null to compute them in the epilogue.
// X null: RMSNorm in front as in rllm_tc_gemm_norm (h, ldh, g, g_dt, eps; T at most 64).
RLLM_API int rllm_tc_gemm_qkv_rope(const void* X, long long ldx, const float* h, long long ldh, const void* g,
                                   int g_dt, float eps, const void* W, void* QKV, long long ldc, int T,
                                   int K, const int* positions, const float* inv_freq, const void* cos_sin,
                                   const int* slots, void* kcache, void* vcache, int nh, int nkv, int hd, int page_size,
                                   int rot_dim, int allow_split, int* err, int sm_count, void* stream) {
  if (hd <= 0 || BM % hd || rot_dim % 2 || rot_dim > hd || rot_dim < 0 || nh <= 0 || nkv <= 0 || page_size <= 0)
    return ERR_BAD_SIZE;
  RopeArgs r;
  r.positions = positions; r.inv_freq = inv_freq; r.cos_sin = (const float2*)cos_sin; r.slots = slots; r.kcache = (bf16*)kcache;
  r.vcache = (bf16*)vcache; r.nh = nh; r.nkv = nkv; r.hd = hd; r.page_size = page_size; r.rot_dim = rot_dim;
  NormArgs nm;
  const bool fused = X == nullptr;
  if (fused) {
    if (!h || !g || (g_dt != DT_F32 && g_dt != DT_BF16)) return ERR_BAD_SIZE;
    nm.h = h; nm.ldh = ldh; nm.rows = nullptr; nm.g = g; nm.g_is_bf16 = g_dt == DT_BF16; nm.eps = eps;
  }
  return run(EPI_QKV_ROPE, X, ldx, fused ? &nm : nullptr, W, QKV, ldc, T, (nh + 2 * nkv) * hd, K, allow_split, err,
             sm_count, &r, stream);
}
