// Weight-streaming matrix product for steps of at most 8 tokens (decoding at small batch):
//     C[T, N] = X[T, K] * W[N, K]^T,  T <= 8
//
// At these sizes the product is a read of W and nothing else, so the kernel is built around the
// read. A job is a slab of 16 weight rows (or a pair of slabs whose results meet in the epilogue:
// gate and up rows for SwiGLU, a rotary pair d / d + hd/2 of a head for the q/k/v projection).
// The 16 warps of a CTA split K between them; every warp copies its own pieces of the slab
// (16 rows x 128 values of K = 4 KB a chunk) with cp.async into a ring of its own and multiplies with
// mma.sync m16n8k16: weights are the A operand (16 rows), the tokens the B operand (n = 8). A lane's
// 16-byte fragment read holds 8 consecutive values of K of one row; the contraction index is permuted
// the same way on both operands, so no shuffle or ldmatrix is needed. The warps' partial sums meet in
// shared memory, are added in warp order, and the epilogue runs one thread per output. There are no
// thread-block clusters, no tensor memory and no barriers other than two __syncthreads a batch of
// jobs: what a 16 KB tcgen05 tile costs in fixed work (allocation, mbarrier hand-overs, 50 ns an
// issued MMA, the push to the column's owner) is what a step of 8 tokens spent its time on. The
// tcgen05 kernels of tc_gemm.cu take over from 9 tokens.
//
// The token operand is small and the same for every job, so a warp builds its fragments once,
// after the predecessor has finished, and keeps them in registers (K up to 8,192), or fetches them
// chunk by chunk, one chunk ahead (longer K). With RMSNorm in front the fragments are
// bf16(h * g) built from the float residual stream, the warps add up h^2 on the way and the
// epilogue multiplies by rsqrt(mean + eps), as the tcgen05 kernel does.
//
// Programmatic dependent launch: the kernel lets its successor start at once and copies its first
// weight chunks (which no kernel writes) before it waits for its predecessor; a successor's CTA takes an
// SM as soon as this kernel's CTA there has left.
//
// Reference counterparts: matvec_bf16 (src/gpu/cuda/shaders/matmul.cu:49-77), fused_gate_up_swiglu
// (moe.cu:86-147), rms_norm (rms_norm.cu:78-115), rotary_embedding (rope.cu:62-77),
// copy_to_paged_kv_cache (attention.cu:295-300).
#include "common.cuh"

using namespace rllm;

namespace {

enum : int { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU = 3, EPI_QKV_ROPE = 4 };

constexpr int NT = 8;                            // token columns of the MMA
constexpr int CK = 128;                          // values of K per chunk: 256 bytes of each of 16 rows
constexpr int CHUNK_BYTES = 16 * CK * 2;         // 4 KB
constexpr int MAX_RESIDENT = 4;                  // chunks per warp whose token fragments stay in registers

// A CTA is 16 warps with three chunks each in flight: 192 KB on the way per SM. Bytes in flight are what
// the rate hangs on: 8 warps with two chunks each, which would leave room for the next kernel's CTAs on
// the same SM, ran the decode step 24 % slower (measured on a B200, Llama 3.2 1B shapes, 8 tokens).
struct Cfg {
  static constexpr int WARPS = 16;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int RING = 3;                 // chunks in flight per warp
  static constexpr int BATCH = 2;                // jobs whose partial sums lie in shared memory together
  static constexpr int RING_BYTES = WARPS * RING * CHUNK_BYTES;
  static constexpr int RED_FLOATS = BATCH * 2 * WARPS * 16 * NT;
  static constexpr int SMEM_BYTES = RING_BYTES + RED_FLOATS * 4;
};

struct RopeArgs {
  const int* positions;     // [T]
  const float* inv_freq;    // [hd / 2]
  const float2* cos_sin;    // [T][hd / 2] or null: computed here
  const int* slots;         // [T] page * page_size + offset, < 0: no write; may be null
  bf16* kcache;             // [pages][nkv][page_size][hd]
  bf16* vcache;
  int nh, nkv, hd, page_size;
};

struct Params {
  const bf16* W;            // [rows][K]
  int N, K;                 // output features (SwiGLU: of one half), inner size
  int up_row0;              // SwiGLU: first weight row of the up half
  const bf16* x;            // token operand [T][K], row stride ldx (NORM: unused)
  long long ldx;
  const float* h;           // NORM: float rows, stride ldh; row of token t = rows ? rows[t] : t
  long long ldh;
  const int* rows;
  const void* g;            // norm weight [K]
  int g_is_bf16;
  float eps;
  void* C;                  // output [T][N] (type by epilogue), row stride ldc
  long long ldc;
  int T;
  int njobs;
  int nchw;                 // chunks per warp and tile
  RopeArgs rope;
};

__device__ __forceinline__ void cp16_zfill(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Where token column `col` of row `row` lies within the row's 8 floats of a warp's partial sums: rows four
// apart would meet the same bank, so the column index is flipped by an even number that differs for them (a
// pair of columns 2t, 2t + 1 stays a pair).
__device__ __forceinline__ int red_col(int row, int col) { return col ^ (((row >> 2) & 3) << 1); }

// first weight row of a job's tile
template <int EPI>
__device__ __forceinline__ int tile_row0(const Params& p, int job, int tile) {
  if (EPI == EPI_SWIGLU) return job * 16 + (tile ? p.up_row0 : 0);
  if (EPI == EPI_QKV_ROPE) {
    const int per_head = p.rope.hd >> 5;               // jobs per head: hd / 32
    const int head = job / per_head, sub = job % per_head;
    return head * p.rope.hd + sub * 16 + (tile ? (p.rope.hd >> 1) : 0);
  }
  return job * 16;
}

// This lane's token fragment for one chunk: token g, k = k0 + 32 kb + 8 t .. + 7 for kb = 0..3
// (zeros beyond T or K). NORM: bf16(h * g); the squares of h are added to `ss`.
template <bool NORM>
__device__ __forceinline__ void load_frag(const Params& p, int k0, int g, int t, uint4 (&b)[4], float& ss) {
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    const int k = k0 + 32 * kb + 8 * t;
    b[kb] = make_uint4(0u, 0u, 0u, 0u);
    if (g < p.T && k < p.K) {
      if (NORM) {
        const float* hr = p.h + (size_t)(p.rows ? p.rows[g] : g) * p.ldh + k;
        const float4 a = __ldcg(reinterpret_cast<const float4*>(hr));
        const float4 c = __ldcg(reinterpret_cast<const float4*>(hr + 4));
        float gv[8];
        if (p.g_is_bf16) {
          const uint4 gw = __ldg(reinterpret_cast<const uint4*>((const bf16*)p.g + k));
          const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gw);
#pragma unroll
          for (int e = 0; e < 4; ++e) { gv[2 * e] = __low2float(g2[e]); gv[2 * e + 1] = __high2float(g2[e]); }
        } else {
          const float4 g0 = __ldg(reinterpret_cast<const float4*>((const float*)p.g + k));
          const float4 g1 = __ldg(reinterpret_cast<const float4*>((const float*)p.g + k + 4));
          gv[0] = g0.x; gv[1] = g0.y; gv[2] = g0.z; gv[3] = g0.w;
          gv[4] = g1.x; gv[5] = g1.y; gv[6] = g1.z; gv[7] = g1.w;
        }
        ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
        ss = fmaf(c.x, c.x, ss); ss = fmaf(c.y, c.y, ss); ss = fmaf(c.z, c.z, ss); ss = fmaf(c.w, c.w, ss);
        b[kb].x = pack2(a.x * gv[0], a.y * gv[1]); b[kb].y = pack2(a.z * gv[2], a.w * gv[3]);
        b[kb].z = pack2(c.x * gv[4], c.y * gv[5]); b[kb].w = pack2(c.z * gv[6], c.w * gv[7]);
      } else {
        b[kb] = __ldcg(reinterpret_cast<const uint4*>(p.x + (size_t)g * p.ldx + k));
      }
    }
  }
}

// NCH: chunks per warp and tile whose token fragments stay in registers (1..4), or 0: any number,
// fragments fetched chunk by chunk (no norm in front then: the squares would be counted per job).
//
// How a chunk travels. One cp.async instruction of a warp copies two rows, 256 contiguous bytes of
// each (lanes 0-15 the even row, 16-31 the odd one): long runs are what the memory system delivers
// fastest (measured on a B200 over this layer's weights: 4.6 TB/s with 64-byte pieces of eight rows
// an instruction, 6.9 TB/s this way). In shared memory a row keeps its 256 bytes together, the
// 16-byte units of odd rows with bit 2 of their index flipped, so that the fragment reads (a quarter
// warp = two rows x four units) meet no bank twice. A lane reads what other lanes copied: every lane
// waits for its own copies, then the warp meets (__syncwarp) before the reads and again before the
// slot is refilled.
template <int EPI, bool NORM, int NCH>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
stream_gemm_kernel(const Params p) {
  typedef Cfg C;
  constexpr int WARPS = C::WARPS, RING = C::RING, BATCH = C::BATCH, THREADS = C::THREADS;
  constexpr int TILES = (EPI == EPI_SWIGLU || EPI == EPI_QKV_ROPE) ? 2 : 1;
  static_assert(!(NORM && NCH == 0), "norm in front needs resident fragments");
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float ss_red[WARPS][NT];
  float* red = reinterpret_cast<float*>(smem + C::RING_BYTES);    // [job of batch][tile][warp][row][token]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * (RING * CHUNK_BYTES);
  const int nchw = NCH ? NCH : p.nchw;
  const int my_jobs = p.njobs > (int)blockIdx.x ? (p.njobs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  pdl_launch();

  // ---- producer side of this warp: the chunks in the order they are used
  int pj = 0, ptile = 0, pci = 0, pslot = 0;
  const int crow = lane >> 4, cunit = lane & 15;           // this lane's part of a copy instruction
  auto produce = [&]() {
    if (pj < my_jobs) {
      const int job = blockIdx.x + pj * gridDim.x;
      const int row0 = tile_row0<EPI>(p, job, ptile);
      const int k = (warp * nchw + pci) * CK + 8 * cunit;
      const bool valid = k < p.K;
      const bf16* src = valid ? p.W + (size_t)(row0 + crow) * p.K + k : p.W;
      const uint32_t dst = ring + pslot * CHUNK_BYTES + crow * 256 + ((cunit ^ (crow << 2)) << 4);
#pragma unroll
      for (int i = 0; i < 8; ++i) cp16_zfill(dst + i * 512, valid ? src + (size_t)(2 * i) * p.K : p.W, valid);
      if (++pci == nchw) { pci = 0; if (++ptile == TILES) { ptile = 0; ++pj; } }
    }
    cp_commit();
    pslot = pslot + 1 == RING ? 0 : pslot + 1;
  };
#pragma unroll
  for (int i = 0; i < RING; ++i) produce();      // weights do not depend on the kernel before this one

  pdl_wait();                                    // the token operand does, and nothing is written before

  // ---- the token fragments
  uint4 bres[NCH ? NCH : 1][4];
  float ss = 0.f;
  if (NCH) {
#pragma unroll
    for (int ci = 0; ci < (NCH ? NCH : 1); ++ci) load_frag<NORM>(p, (warp * nchw + ci) * CK, g, t, bres[ci], ss);
    if (NORM) {
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      if (t == 0) ss_red[warp][g] = ss;
    }
  }

  int cslot = 0;
  // rows g and g + 8 have the parity of g: one key for both
  const uint32_t frag_off = (uint32_t)(g * 256), frag_key = (uint32_t)((g & 1) << 2);
  auto consume = [&](float (&acc)[4], const uint4 (&b)[4]) {
    cp_wait<RING - 1>();
    __syncwarp();
    const uint32_t src = ring + cslot * CHUNK_BYTES + frag_off;
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const uint32_t a = src + ((((uint32_t)(4 * kb + t)) ^ frag_key) << 4);
      uint4 lo, hi;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "r"(a));
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "r"(a + 8 * 256));
      mma16816(acc, lo.x, hi.x, lo.y, hi.y, b[kb].x, b[kb].y);
      mma16816(acc, lo.z, hi.z, lo.w, hi.w, b[kb].z, b[kb].w);
    }
    cslot = cslot + 1 == RING ? 0 : cslot + 1;
    __syncwarp();                                // every lane has read the slot that is refilled now
    produce();
  };
  for (int batch0 = 0; batch0 < my_jobs; batch0 += BATCH) {
    const int nb = min(BATCH, my_jobs - batch0);
    for (int jb = 0; jb < nb; ++jb) {
#pragma unroll
      for (int tile = 0; tile < TILES; ++tile) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (NCH) {
#pragma unroll
          for (int ci = 0; ci < (NCH ? NCH : 1); ++ci) consume(acc, bres[ci]);
        } else {
          uint4 bcur[4], bnext[4];
          float unused = 0.f;
          load_frag<false>(p, (warp * nchw) * CK, g, t, bcur, unused);
          for (int ci = 0; ci < nchw; ++ci) {
            if (ci + 1 < nchw) load_frag<false>(p, (warp * nchw + ci + 1) * CK, g, t, bnext, unused);
            consume(acc, bcur);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) bcur[kb] = bnext[kb];
          }
        }
        // (a row's 8 token columns are stored with their index flipped by the row's group of four, red_col:
        // the epilogue's threads, 16 rows of one token side by side, then meet 16 different banks)
        float* r = red + ((size_t)((jb * 2 + tile) * WARPS + warp)) * (16 * NT);
        *reinterpret_cast<float2*>(r + g * NT + red_col(g, 2 * t)) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(r + (g + 8) * NT + red_col(g + 8, 2 * t)) = make_float2(acc[2], acc[3]);
      }
    }
    __syncthreads();
    // ---- the warps' parts in warp order, then the epilogue: thread = (job of batch, token, row of slab)
    for (int e = threadIdx.x; e < nb * 128; e += THREADS) {
      const int jb = e >> 7, tok = (e >> 4) & 7, r = e & 15;
      if (tok >= p.T) continue;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        s0 += red[(size_t)((jb * 2) * WARPS + w) * (16 * NT) + r * NT + red_col(r, tok)];
        if (TILES == 2) s1 += red[(size_t)((jb * 2 + 1) * WARPS + w) * (16 * NT) + r * NT + red_col(r, tok)];
      }
      if (NORM) {
        float sq = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) sq += ss_red[w][tok];
        const float rs = rsqrtf(sq / (float)p.K + p.eps);
        s0 *= rs; s1 *= rs;
      }
      const int job = blockIdx.x + (batch0 + jb) * gridDim.x;
      if (EPI == EPI_QKV_ROPE) {
        const RopeArgs& ra = p.rope;
        const int half = ra.hd >> 1;
        const int n0 = tile_row0<EPI>(p, job, 0) + r, n1 = n0 + half;
        const int head = n0 / ra.hd, d = n0 % ra.hd;          // d < half
        float o0 = s0, o1 = s1;
        if (head < ra.nh + ra.nkv) {
          float sn, cs;
          if (ra.cos_sin) { const float2 v = ra.cos_sin[(size_t)tok * half + d]; cs = v.x; sn = v.y; }
          else sincosf((float)ra.positions[tok] * ra.inv_freq[d], &sn, &cs);
          o0 = s0 * cs - s1 * sn;
          o1 = s0 * sn + s1 * cs;
        }
        const bf16 b0 = __float2bfloat16_rn(o0), b1 = __float2bfloat16_rn(o1);
        bf16* c = (bf16*)p.C + (size_t)tok * p.ldc;
        c[n0] = b0; c[n1] = b1;
        if (head >= ra.nh && ra.slots) {
          const int slot = ra.slots[tok];
          if (slot >= 0) {
            const int page = slot / ra.page_size, off = slot % ra.page_size;
            const bool is_k = head < ra.nh + ra.nkv;
            const int kvh = is_k ? head - ra.nh : head - ra.nh - ra.nkv;
            bf16* dst = (is_k ? ra.kcache : ra.vcache) + (((size_t)page * ra.nkv + kvh) * ra.page_size + off) * ra.hd;
            dst[d] = b0; dst[d + half] = b1;
          }
        }
      } else {
        const size_t o = (size_t)tok * p.ldc + job * 16 + r;
        if (EPI == EPI_STORE) ((bf16*)p.C)[o] = __float2bfloat16_rn(s0);
        else if (EPI == EPI_STORE_F32) ((float*)p.C)[o] = s0;
        else if (EPI == EPI_ACCUM_F32) ((float*)p.C)[o] += s0;
        else if (EPI == EPI_SWIGLU) ((bf16*)p.C)[o] = __float2bfloat16_rn(s0 / (1.f + expf(-s0)) * s1);
      }
    }
    if (batch0 + BATCH < my_jobs) __syncthreads();      // the parts are read before the next batch overwrites them
  }
  cp_wait<0>();
}

// ------------------------------------------------------------------------------------ host side
template <int EPI, bool NORM, int NCH>
int launch(const Params& p, int ctas, cudaStream_t s) {
  typedef Cfg C;
  static bool configured[64] = {};
  if (allow_dynamic_smem(stream_gemm_kernel<EPI, NORM, NCH>, C::SMEM_BYTES, configured)) return -5;
  return launch_ex(stream_gemm_kernel<EPI, NORM, NCH>, dim3(ctas), dim3(C::THREADS), C::SMEM_BYTES, s, 1, p);
}

template <int EPI, bool NORM>
int launch_nch(const Params& p, int ctas, cudaStream_t s) {
  switch (p.nchw) {
    case 1: return launch<EPI, NORM, 1>(p, ctas, s);
    case 2: return launch<EPI, NORM, 2>(p, ctas, s);
    case 3: return launch<EPI, NORM, 3>(p, ctas, s);
    case 4: return launch<EPI, NORM, 4>(p, ctas, s);
  }
  if constexpr (!NORM) return launch<EPI, false, 0>(p, ctas, s);
  return ERR_BAD_SIZE;
}

int chunks_per_warp(int K) { return ((K + CK - 1) / CK + Cfg::WARPS - 1) / Cfg::WARPS; }

// Can the kernel take this problem? The rules the launchers below enforce.
int supported(int epi, bool norm, int T, int N, int K, int hd) {
  if (T < 1 || T > NT || N < 16 || N % 16 || K < 32 || K % 32) return 0;
  if (epi < 0 || epi > EPI_QKV_ROPE) return 0;
  if (norm && (epi == EPI_ACCUM_F32 || chunks_per_warp(K) > MAX_RESIDENT)) return 0;
  if (epi == EPI_QKV_ROPE && (hd < 32 || hd % 32 || N % hd)) return 0;
  return 1;
}

int run(int epi, bool norm, Params& p, int sm_count, cudaStream_t s) {
  if (!supported(epi, norm, p.T, p.N, p.K, p.rope.hd)) return ERR_BAD_SIZE;
  if ((uintptr_t)p.W & 15) return ERR_BAD_ALIGN;
  if (norm) {
    if (p.ldh % 4 || ((uintptr_t)p.h & 15) || ((uintptr_t)p.g & 15)) return ERR_BAD_ALIGN;
  } else if (p.ldx % 8 || ((uintptr_t)p.x & 15)) return ERR_BAD_ALIGN;
  p.njobs = epi == EPI_QKV_ROPE ? p.N / 32 : p.N / 16;
  p.nchw = chunks_per_warp(p.K);
  int ctas = p.njobs < sm_count ? p.njobs : sm_count;
  // A short product between two long ones (the mixer's output product: 64 KB a job) takes two jobs a CTA and so
  // half as many SMs: on the others the successor's CTAs are resident early, with their first weights on
  // the way (measured in the decode step of Llama 3.2 1B: batch 1 1,593 -> 1,660 tok/s, batch 8 9,908 -> 9,948).
  if (epi == EPI_ACCUM_F32 && p.njobs <= sm_count && (size_t)32 * p.K <= 64 * 1024) ctas = (p.njobs + 1) / 2;
  if (norm) {
    switch (epi) {
      case EPI_STORE: return launch_nch<EPI_STORE, true>(p, ctas, s);
      case EPI_STORE_F32: return launch_nch<EPI_STORE_F32, true>(p, ctas, s);
      case EPI_SWIGLU: return launch_nch<EPI_SWIGLU, true>(p, ctas, s);
      case EPI_QKV_ROPE: return launch_nch<EPI_QKV_ROPE, true>(p, ctas, s);
    }
    return ERR_BAD_SIZE;
  }
  switch (epi) {
    case EPI_STORE: return launch_nch<EPI_STORE, false>(p, ctas, s);
    case EPI_STORE_F32: return launch_nch<EPI_STORE_F32, false>(p, ctas, s);
    case EPI_ACCUM_F32: return launch_nch<EPI_ACCUM_F32, false>(p, ctas, s);
    case EPI_SWIGLU: return launch_nch<EPI_SWIGLU, false>(p, ctas, s);
    case EPI_QKV_ROPE: return launch_nch<EPI_QKV_ROPE, false>(p, ctas, s);
  }
  return ERR_BAD_SIZE;
}

}  // namespace

// 1 when rllm_stream_gemm / rllm_stream_gemm_qkv_rope take the problem (T tokens, N output features
// (of one half with SwiGLU), inner size K, norm in front or not; hd: head size, rotary epilogue only).
RLLM_API int rllm_stream_gemm_supported(int epi, int norm, int T, int N, int K, int hd) {
  return supported(epi, norm != 0, T, N, K, hd);
}

// C[T, N] = X W^T for T <= 8. X: bf16 [T, K] with row stride ldx, or null: then X = rmsnorm(h[rows]; g, eps)
// built inside the kernel from float rows h (stride ldh; rows null: row t). W: bf16 [N, K] contiguous
// ([2N, K] for SwiGLU: gate rows, then up rows). Epilogues 0..3 as in rllm_tc_gemm.
RLLM_API int rllm_stream_gemm(int epi, const void* X, long long ldx, const float* h, long long ldh, const int* rows,
                              const void* g, int g_dt, float eps, const void* W, void* Cout, long long ldc,
                              int T, int N, int K, int sm_count, void* stream) {
  if (epi < 0 || epi > EPI_SWIGLU) return ERR_BAD_SIZE;
  const bool norm = X == nullptr;
  if (norm && (!h || !g || (g_dt != DT_F32 && g_dt != DT_BF16))) return ERR_BAD_SIZE;
  Params p = {};
  p.W = (const bf16*)W; p.N = N; p.K = K; p.up_row0 = N; p.x = (const bf16*)X; p.ldx = ldx;
  p.h = h; p.ldh = ldh; p.rows = rows; p.g = g; p.g_is_bf16 = g_dt == DT_BF16; p.eps = eps;
  p.C = Cout; p.ldc = ldc; p.T = T;
  return run(epi, norm, p, sm_count, (cudaStream_t)stream);
}

// The q/k/v projection for T <= 8 with the rotation of q and k (pairs d, d + hd/2 of every head, the
// whole head rotated) and the write of k and v into the paged cache in its epilogue; arguments as in
// rllm_tc_gemm_qkv_rope. Head size a multiple of 32.
RLLM_API int rllm_stream_gemm_qkv_rope(const void* X, long long ldx, const float* h, long long ldh, const void* g,
                                       int g_dt, float eps, const void* W, void* QKV, long long ldc, int T, int K,
                                       const int* positions, const float* inv_freq, const void* cos_sin,
                                       const int* slots, void* kcache, void* vcache, int nh, int nkv, int hd,
                                       int page_size, int sm_count, void* stream) {
  if (hd <= 0 || nh <= 0 || nkv <= 0 || page_size <= 0) return ERR_BAD_SIZE;
  const bool norm = X == nullptr;
  if (norm && (!h || !g || (g_dt != DT_F32 && g_dt != DT_BF16))) return ERR_BAD_SIZE;
  Params p = {};
  p.W = (const bf16*)W; p.N = (nh + 2 * nkv) * hd; p.K = K; p.x = (const bf16*)X; p.ldx = ldx;
  p.h = h; p.ldh = ldh; p.rows = nullptr; p.g = g; p.g_is_bf16 = g_dt == DT_BF16; p.eps = eps;
  p.C = QKV; p.ldc = ldc; p.T = T;
  p.rope.positions = positions; p.rope.inv_freq = inv_freq; p.rope.cos_sin = (const float2*)cos_sin;
  p.rope.slots = slots; p.rope.kcache = (bf16*)kcache; p.rope.vcache = (bf16*)vcache;
  p.rope.nh = nh; p.rope.nkv = nkv; p.rope.hd = hd; p.rope.page_size = page_size;
  return run(EPI_QKV_ROPE, norm, p, sm_count, (cudaStream_t)stream);
}
