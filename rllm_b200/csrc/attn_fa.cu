// Tiled attention over the paged bfloat16 cache on the tensor cores, for prefill portions,
// single decoded tokens and any mix of them in one launch.
//
// The rows of a tile are (query token, query head) pairs of ONE kv head: row r of a sequence
// is token r / G, head kvh*G + r % G (G = heads per kv head), so the G query heads of a group
// share every K/V byte that is loaded. A warp owns 16 rows; a CTA of NWARPS warps shares the
// K/V tiles (64 keys) that cp.async brings into shared memory through the block table, two
// tiles in flight. Scores and the weighted sum use mma.sync m16n8k16 (bf16 in, float
// accumulate); the softmax is the running-maximum form in float with exp2.
// Each row sees keys j <= its own position, and j > position - window when a window is set.
//
// Split-KV (decode): the visible keys of a sequence are cut into `splits` ranges, one CTA
// each, which leave unnormalised partial sums (o, max, sum) in scratch memory; a second
// kernel merges them in split order.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:328-388 of the reference (scale, softmax with
// the maximum subtracted, weighted V, head h -> kv head h / G, window start :337-338). The
// reference's prefill kernel attends inside the chunk only (attention.cu:573-618); here a
// portion also sees what earlier steps left in the cache.
// Cache layout: [page][kv head][offset in page][HD].
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int BN = 64;   // keys per tile

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_addr_x4(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_addr_x4_trans(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ float fast_exp2(float x) {          // exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct FaParams {
  const bf16* q; int q_stride;
  const bf16* kc; const bf16* vc;
  bf16* out; int out_stride;
  const int* cu_q; const int* kv_lens; const int* block_table; int bt_stride;
  int nh, nkv, page_size, page_shift, window, splits;
  float scale_log2e;
  float* part_o;      // [(token * nh + head) * splits + z][HD]
  float* part_ml;     // [(token * nh + head) * splits + z][2]
  long long part_rows;   // rows the two buffers above have: a row index beyond it (a cu_q that names more
                         // tokens than the caller said) is skipped, never written
};

template <int HD, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
fa_paged_kernel(const FaParams p) {
  pdl_launch();
  pdl_wait();
  constexpr int BM = 16 * NWARPS;
  constexpr int CH = HD / 8;            // 16-byte chunks per key row
  constexpr int NT = NWARPS * 32;
  constexpr int KSTEPS = HD / 16;       // k-steps of the score product
  constexpr int DTILES = HD / 8;        // 8-wide output tiles of the weighted sum
  extern __shared__ __align__(128) uint8_t fa_smem[];
  bf16* Ks = reinterpret_cast<bf16*>(fa_smem);               // [2][BN * HD]
  bf16* Vs = Ks + 2 * BN * HD;                               // [2][BN * HD]

  const int seq = blockIdx.z;
  const int kvh = blockIdx.y / p.splits, z = blockIdx.y % p.splits;
  // the last rows of a prompt see the most keys: those tiles start first, the short ones fill in behind
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int G = p.nh / p.nkv;
  const int q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - q0;
  const int kv_len = p.kv_lens[seq];
  const int rows_total = q_len * G;
  if (tile * BM >= rows_total) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, qi = lane & 3;

  // keys this tile can see at all
  const int tok_first = (tile * BM) / G;
  const int tok_last = min(q_len - 1, (tile * BM + BM - 1) / G);
  const int p_min = kv_len - q_len + tok_first, p_max = kv_len - q_len + tok_last;
  int kv_begin = (p.window > 0 && p_min - p.window + 1 > 0) ? p_min - p.window + 1 : 0;
  kv_begin = kv_begin / BN * BN;
  const int kv_end = p_max + 1;
  const int tiles_total = (kv_end - kv_begin + BN - 1) / BN;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int tb = z * tiles_per_split;
  const int te = min(tiles_total, tb + tiles_per_split);

  // this thread's two rows (A: quad, B: quad + 8 of the warp's 16)
  int rowA = tile * BM + warp * 16 + quad, rowB = rowA + 8;
  bool vA = rowA < rows_total, vB = rowB < rows_total;
  const int tokA = vA ? rowA / G : 0, tokB = vB ? rowB / G : 0;
  const int headA = kvh * G + (vA ? rowA % G : 0), headB = kvh * G + (vB ? rowB % G : 0);
  const int posA = kv_len - q_len + tokA, posB = kv_len - q_len + tokB;
  const int loA = (p.window > 0) ? posA - p.window + 1 : 0, loB = (p.window > 0) ? posB - p.window + 1 : 0;

  // Q fragments, straight from global memory
  uint32_t qf[KSTEPS][4];
  {
    const bf16* qa = p.q + (size_t)(q0 + tokA) * p.q_stride + (size_t)headA * HD;
    const bf16* qb = p.q + (size_t)(q0 + tokB) * p.q_stride + (size_t)headB * HD;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d = kk * 16 + qi * 2;
      qf[kk][0] = vA ? *reinterpret_cast<const uint32_t*>(qa + d) : 0u;
      qf[kk][1] = vB ? *reinterpret_cast<const uint32_t*>(qb + d) : 0u;
      qf[kk][2] = vA ? *reinterpret_cast<const uint32_t*>(qa + d + 8) : 0u;
      qf[kk][3] = vB ? *reinterpret_cast<const uint32_t*>(qb + d + 8) : 0u;
    }
  }

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

  // What the 16 rows of this warp can see (the same for all its lanes): a tile wholly inside is
  // taken without a mask, a tile wholly outside is not computed at all.
  const int wrow0 = tile * BM + warp * 16;
  const bool w_active = wrow0 < rows_total;
  const int wpos_min = kv_len - q_len + (w_active ? wrow0 / G : 0);
  const int wpos_max = kv_len - q_len + (w_active ? min(rows_total - 1, wrow0 + 15) / G : 0);
  const int wlo_min = p.window > 0 ? wpos_min - p.window + 1 : 0;     // smallest first visible key of a row
  const int wlo_max = p.window > 0 ? wpos_max - p.window + 1 : 0;     // largest
  const bool rows_full = wrow0 + 15 < rows_total;

  // shared-memory addresses of this lane's ldmatrix rows, swizzle included (they do not depend on the tile)
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks), vs_base = (uint32_t)__cvta_generic_to_shared(Vs);
  const int mat = lane >> 3, rr = lane & 7;
  uint32_t koff[KSTEPS], voff[DTILES / 2];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk)
    koff[kk] = (uint32_t)((((mat >> 1) * 8 + rr) * HD + (((2 * kk + (mat & 1)) ^ rr) * 8)) * 2);
#pragma unroll
  for (int dp = 0; dp < DTILES / 2; ++dp)
    voff[dp] = (uint32_t)((((mat & 1) * 8 + rr) * HD + (((2 * dp + (mat >> 1)) ^ rr) * 8)) * 2);

  const int* bt = p.block_table + (size_t)seq * p.bt_stride;
  const int pshift = p.page_shift;                       // log2(page_size), or < 0 when it is no power of two
  auto load_tile = [&](int t, int buf) {
    const int j0 = kv_begin + t * BN;
    const uint32_t kd = ks_base + (uint32_t)(buf * BN * HD * 2), vd = vs_base + (uint32_t)(buf * BN * HD * 2);
#pragma unroll
    for (int c = threadIdx.x; c < BN * CH; c += NT) {
      const int r = c / CH, ch = c % CH;
      const int j = j0 + r;
      bool ok = j < kv_len;
      const int pg = pshift >= 0 ? (j >> pshift) : j / p.page_size;
      const int off = pshift >= 0 ? (j & (p.page_size - 1)) : j % p.page_size;
      int page = ok ? __ldg(bt + pg) : -1;
      ok = ok && page >= 0;
      const size_t src = ok ? ((((size_t)page * p.nkv + kvh) * p.page_size + off) * HD + ch * 8) : 0;
      const uint32_t dst = (uint32_t)((r * HD + ((ch ^ (r & 7)) * 8)) * 2);
      const int n = ok ? 16 : 0;                          // 0 bytes read: the 16 bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd + dst), "l"(p.kc + src), "r"(n) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd + dst), "l"(p.vc + src), "r"(n) : "memory");
    }
  };

  if (tb < te) load_tile(tb, 0);
  cp_async_commit();

  for (int t = tb; t < te; ++t) {
    const int buf = (t - tb) & 1;
    if (t + 1 < te) load_tile(t + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kt = ks_base + (uint32_t)(buf * BN * HD * 2);
    const uint32_t vt = vs_base + (uint32_t)(buf * BN * HD * 2);
    const int j0 = kv_begin + t * BN;

    if (w_active && j0 <= wpos_max && j0 + BN - 1 >= wlo_min) {
      // ---- scores S = Q K^T : 16 rows x 64 keys; the K fragments of a k-step are fetched together
      float s[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t b[BN / 16][4];
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) ldsm_addr_x4(b[np], kt + koff[kk] + (uint32_t)(np * 16 * HD * 2));
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          mma_bf16(s[2 * np], qf[kk], b[np][0], b[np][1]);
          mma_bf16(s[2 * np + 1], qf[kk], b[np][2], b[np][3]);
        }
      }
      // ---- mask (only a tile at an edge of what the warp sees), running maximum
      if (j0 + BN - 1 > wpos_min || j0 < wlo_max || !rows_full) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = j0 + nt * 8 + qi * 2 + e;
            if (!(vA && j <= posA && j >= loA)) s[nt][e] = -INFINITY;
            if (!(vB && j <= posB && j >= loB)) s[nt][2 + e] = -INFINITY;
          }
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
        mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      // the running maximum lives in the exp2 domain (the scale is positive: it commutes with max)
      const float sl = p.scale_log2e;
      const float mnA = fmaxf(mA, mxA * sl), mnB = fmaxf(mB, mxB * sl);
      const float useA = (mnA == -INFINITY) ? 0.f : mnA, useB = (mnB == -INFINITY) ? 0.f : mnB;
      if (__any_sync(0xffffffffu, mnA != mA || mnB != mB)) {      // a new maximum somewhere: rescale
        const float corrA = fast_exp2(mA - useA), corrB = fast_exp2(mB - useB);     // exp2(-inf) = 0
        lA *= corrA; lB *= corrB;
#pragma unroll
        for (int i = 0; i < DTILES; ++i) { o[i][0] *= corrA; o[i][1] *= corrA; o[i][2] *= corrB; o[i][3] *= corrB; }
        mA = mnA; mB = mnB;
      }
      // ---- probabilities (as bf16 A fragments) and the weighted sum O += P V
#pragma unroll
      for (int kb = 0; kb < BN / 16; ++kb) {
        uint32_t vb[DTILES / 2][4];
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) ldsm_addr_x4_trans(vb[dp], vt + voff[dp] + (uint32_t)(kb * 16 * HD * 2));
        uint32_t a[4];
        {
          const float p0 = fast_exp2(fmaf(s[2 * kb][0], sl, -useA)), p1 = fast_exp2(fmaf(s[2 * kb][1], sl, -useA));
          const float p2 = fast_exp2(fmaf(s[2 * kb][2], sl, -useB)), p3 = fast_exp2(fmaf(s[2 * kb][3], sl, -useB));
          const float p4 = fast_exp2(fmaf(s[2 * kb + 1][0], sl, -useA)), p5 = fast_exp2(fmaf(s[2 * kb + 1][1], sl, -useA));
          const float p6 = fast_exp2(fmaf(s[2 * kb + 1][2], sl, -useB)), p7 = fast_exp2(fmaf(s[2 * kb + 1][3], sl, -useB));
          lA += p0 + p1 + p4 + p5;
          lB += p2 + p3 + p6 + p7;
          a[0] = pack_bf16(p0, p1); a[1] = pack_bf16(p2, p3);
          a[2] = pack_bf16(p4, p5); a[3] = pack_bf16(p6, p7);
        }
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          mma_bf16(o[2 * dp], a, vb[dp][0], vb[dp][1]);
          mma_bf16(o[2 * dp + 1], a, vb[dp][2], vb[dp][3]);
        }
      }
    }
    __syncthreads();       // everyone is done with this buffer before it is refilled
  }
  cp_async_wait<0>();

  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);

  if (p.splits == 1) {
    const float iA = lA > 0.f ? 1.f / lA : 0.f, iB = lB > 0.f ? 1.f / lB : 0.f;
    bf16* oa = p.out + (size_t)(q0 + tokA) * p.out_stride + (size_t)headA * HD;
    bf16* ob = p.out + (size_t)(q0 + tokB) * p.out_stride + (size_t)headB * HD;
#pragma unroll
    for (int dn = 0; dn < DTILES; ++dn) {
      const int d = dn * 8 + qi * 2;
      if (vA) *reinterpret_cast<uint32_t*>(oa + d) = pack_bf16(o[dn][0] * iA, o[dn][1] * iA);
      if (vB) *reinterpret_cast<uint32_t*>(ob + d) = pack_bf16(o[dn][2] * iB, o[dn][3] * iB);
    }
  } else {
    const size_t ia = ((size_t)(q0 + tokA) * p.nh + headA) * p.splits + z;
    const size_t ib = ((size_t)(q0 + tokB) * p.nh + headB) * p.splits + z;
    vA = vA && ia < (size_t)p.part_rows;
    vB = vB && ib < (size_t)p.part_rows;
#pragma unroll
    for (int dn = 0; dn < DTILES; ++dn) {
      const int d = dn * 8 + qi * 2;
      if (vA) *reinterpret_cast<float2*>(p.part_o + ia * HD + d) = make_float2(o[dn][0], o[dn][1]);
      if (vB) *reinterpret_cast<float2*>(p.part_o + ib * HD + d) = make_float2(o[dn][2], o[dn][3]);
    }
    if (qi == 0) {
      if (vA) { p.part_ml[ia * 2] = mA; p.part_ml[ia * 2 + 1] = lA; }
      if (vB) { p.part_ml[ib * 2] = mB; p.part_ml[ib * 2 + 1] = lB; }
    }
  }
}

// Merge the partial sums of the splits, in split order: one block per (token, head).
template <int HD>
__global__ void fa_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  bf16* __restrict__ out, int out_stride, int nh, int splits) {
  pdl_launch();
  pdl_wait();
  const int th = blockIdx.x;                 // token * nh + head
  const int token = th / nh, head = th % nh;
  const float* ml = part_ml + (size_t)th * splits * 2;
  float M = -INFINITY;
  for (int z = 0; z < splits; ++z) M = fmaxf(M, ml[2 * z]);
  float L = 0.f;
  for (int z = 0; z < splits; ++z) L += (ml[2 * z] == -INFINITY) ? 0.f : ml[2 * z + 1] * exp2f(ml[2 * z] - M);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; ++z) {
      if (ml[2 * z] == -INFINITY) continue;
      acc += part_o[((size_t)th * splits + z) * HD + d] * exp2f(ml[2 * z] - M);
    }
    out[(size_t)token * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD, int NWARPS>
int launch_fa(const FaParams& p, int num_seqs, int max_rows, cudaStream_t s) {
  constexpr int BM = 16 * NWARPS;
  constexpr int SMEM = 4 * BN * HD * 2;
  static bool configured[64] = {};             // the attribute belongs to a device's copy of the kernel
  if (allow_dynamic_smem(fa_paged_kernel<HD, NWARPS>, SMEM, configured)) return -5;
  dim3 grid((max_rows + BM - 1) / BM, p.nkv * p.splits, num_seqs);
  if (grid.y > 65535 || grid.z > 65535) return ERR_TOO_LARGE;
  return launch_ex(fa_paged_kernel<HD, NWARPS>, grid, dim3(NWARPS * 32), SMEM, s, 1, p);
}

}  // namespace

// q: [T, ...] bf16 rows with stride q_stride, head h at h*hd; out likewise. cu_q [S+1], kv_lens [S],
// block_table [S, bt_stride]. max_q_len: the longest portion in the batch (sizes the grid).
// splits > 1 needs part_o [T*nh*splits*hd] and part_ml [T*nh*splits*2] floats of scratch.
RLLM_API int rllm_attention_fa(const void* q, int q_stride, const void* kcache, const void* vcache, void* out,
                               int out_stride, const int* cu_q, const int* kv_lens, const int* block_table,
                               int bt_stride, int num_seqs, int num_tokens, int max_q_len, int nh, int nkv,
                               int hd, int page_size, float scale, int window, int splits, float* part_o,
                               float* part_ml, void* stream) {
  if (num_seqs <= 0 || num_tokens <= 0) return 0;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || page_size <= 0) return ERR_BAD_SIZE;
  if (q_stride % 2 || out_stride % 2 || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) ||
      ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return ERR_BAD_ALIGN;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!part_o || !part_ml)) return ERR_BAD_SIZE;
  FaParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.kc = (const bf16*)kcache; p.vc = (const bf16*)vcache;
  p.out = (bf16*)out; p.out_stride = out_stride; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.block_table = block_table; p.bt_stride = bt_stride; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
  p.window = window; p.splits = splits; p.scale_log2e = scale * 1.4426950408889634f;
  p.page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) { p.page_shift = 0; while ((1 << p.page_shift) < page_size) ++p.page_shift; }
  p.part_o = part_o; p.part_ml = part_ml;
  p.part_rows = (long long)num_tokens * nh * splits;
  cudaStream_t s = (cudaStream_t)stream;
  const int G = nh / nkv;
  const int max_rows = max_q_len * G;
  int rc;
  if (max_rows <= 16) rc = hd == 64 ? launch_fa<64, 1>(p, num_seqs, max_rows, s) : launch_fa<128, 1>(p, num_seqs, max_rows, s);
  else rc = hd == 64 ? launch_fa<64, 4>(p, num_seqs, max_rows, s) : launch_fa<128, 4>(p, num_seqs, max_rows, s);
  if (rc || splits == 1) return rc;
  const int blocks = num_tokens * nh;
  if (hd == 64)
    return launch_ex(fa_combine_kernel<64>, dim3(blocks), dim3(64), 0, s, 1, (const float*)part_o,
                     (const float*)part_ml, (bf16*)out, out_stride, nh, splits);
  return launch_ex(fa_combine_kernel<128>, dim3(blocks), dim3(128), 0, s, 1, (const float*)part_o,
                   (const float*)part_ml, (bf16*)out, out_stride, nh, splits);
}

// ------------------------------------------------------------------------------------------
// Split-key attention for callers that cannot allocate device memory (see attn_fa_noalloc.h).
// Same kernels as rllm_attention_fa; the partial sums of the key ranges go to a fixed array
// inside this library instead of buffers the caller would have to allocate.
// ------------------------------------------------------------------------------------------
#include "attn_fa_noalloc.h"
#include <mutex>

// One copy per GPU that loads this library, held until the process exits:
// partial outputs first, then the (maximum, sum) pairs.
static __device__ __align__(256) float g_noalloc_scratch[RLLM_NOALLOC_PART_O_FLOATS + RLLM_NOALLOC_PART_ML_FLOATS];

namespace {

constexpr size_t NOALLOC_O_FLOATS = RLLM_NOALLOC_PART_O_FLOATS;
constexpr size_t NOALLOC_ML_FLOATS = RLLM_NOALLOC_PART_ML_FLOATS;
constexpr int NOALLOC_MAX_DEVICES = 64;

// In host code `g_noalloc_scratch` is only a handle; the address a kernel can use is asked
// for once per device, with that device current, and kept here.
float* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {nullptr};
std::mutex g_noalloc_mu;

int noalloc_scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    cudaGetLastError();
    return -5;
  }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_addr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return -5;
    }
    g_noalloc_addr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_addr[dev];
  return 0;
}

}  // namespace

RLLM_API int rllm_attention_fa_noalloc(const void* q, int q_stride, const void* kcache, const void* vcache,
                                       void* out, int out_stride, const int* cu_q, const int* kv_lens,
                                       const int* block_table, int bt_stride, int num_seqs, int num_tokens,
                                       int max_q_len, int nh, int nkv, int hd, int page_size, float scale,
                                       int window, int splits, void* stream) {
  if (num_seqs <= 0 || num_tokens <= 0) return 0;
  if (splits < 1) splits = 1;
  if (nh <= 0 || hd <= 0) return ERR_BAD_SIZE;
  const size_t rows = (size_t)num_tokens * (size_t)nh * (size_t)splits;
  if (splits > 1 && (rows * (size_t)hd > NOALLOC_O_FLOATS || rows * 2 > NOALLOC_ML_FLOATS))
    return ERR_TOO_LARGE;                       // beyond the fixed scratch: refuse, never overrun
  float* scratch = nullptr;
  const int rc = noalloc_scratch_address(&scratch);
  if (rc) return rc;
  // Every (token, head, range) slot that the merge reads is written by the first kernel of the
  // same call, so nothing of an earlier call's contents is ever read and nothing needs clearing.
  return rllm_attention_fa(q, q_stride, kcache, vcache, out, out_stride, cu_q, kv_lens, block_table,
                           bt_stride, num_seqs, num_tokens, max_q_len, nh, nkv, hd, page_size, scale, window,
                           splits, scratch, scratch + NOALLOC_O_FLOATS, stream);
}
