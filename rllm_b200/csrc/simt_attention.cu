// Paged attention on the CUDA cores for any mix of prompt portions and single
// decoded tokens, both storage types, all arithmetic in float.
//
// One warp per (query token, query head). The token's sequence and absolute
// position say which keys it sees: j in [max(0, pos - window + 1), pos] of that
// sequence's block table (window <= 0: all keys from 0). Keys are taken 32 at a
// time in position order with a running maximum and sum, so the result of a
// query depends only on its position and the cache contents, never on how the
// tokens were cut into steps or what else is in the batch.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:328-388 (scores, softmax with the
// maximum subtracted, weighted sum of V; query head h reads KV head h / (nh/nkv)).
// Unlike the reference's prefill kernel (attention.cu:573-618) a prompt portion
// also attends the keys that earlier steps left in the cache.
// Cache layout: [page][kv head][offset in page][hd].
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T> struct Vec16 {};   // 16-byte vector of T
template <> struct Vec16<float> { static constexpr int N = 4; typedef float4 V; };
template <> struct Vec16<bf16> { static constexpr int N = 8; typedef uint4 V; };

__device__ __forceinline__ float dot_vec(const float4& k, const float* q) {
  return k.x * q[0] + k.y * q[1] + k.z * q[2] + k.w * q[3];
}
__device__ __forceinline__ float dot_vec(const uint4& k, const float* q) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&k);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    s = fmaf(f.x, q[2 * i], s);
    s = fmaf(f.y, q[2 * i + 1], s);
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ kcache,
                            const T* __restrict__ vcache, T* __restrict__ out, int out_stride,
                            const int* __restrict__ token_seq, const int* __restrict__ positions,
                            const int* __restrict__ block_table, int bt_stride, int n_tokens,
                            int nh, int nkv, int hd, int page_size, float scale, int window) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[WARPS][MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * WARPS + warp;
  if (gw >= (long long)n_tokens * nh) return;
  const int t = (int)(gw / nh), h = (int)(gw % nh);
  const int kvh = h / (nh / nkv);
  const int seq = token_seq[t];
  const int pos = positions[t];
  const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* bt = block_table + (size_t)seq * bt_stride;

  const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(qp[d]) * scale;
  __syncwarp();

  constexpr int NACC = MAX_HD / 32;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  typedef typename Vec16<T>::V V;
  constexpr int VN = Vec16<T>::N;

  for (int base = start; base <= pos; base += 32) {
    const int j = base + lane;
    bool valid = j <= pos;
    float s = -INFINITY;
    long long row = 0;       // element offset of this lane's key/value row
    const int page = valid ? bt[j / page_size] : -1;
    valid = valid && page >= 0;            // a table entry without a page (given back, or refused by a check): not read
    if (valid) {
      row = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * hd;
      const V* kp = reinterpret_cast<const V*>(kcache + row);
      float dsum = 0.f;
      for (int c = 0; c < hd / VN; ++c) dsum += dot_vec(kp[c], &qs[warp][c * VN]);
      s = dsum;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);          // first chunk: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    const int cnt = min(32, pos - base + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long rj = __shfl_sync(0xffffffffu, row, jj);
      const T* vp = vcache + rj;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vp[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* op = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

// q: [n_tokens, ...] with row stride q_stride (elements), head h at h*hd; out likewise.
// token_seq[t]: row of block_table the token belongs to; positions[t]: absolute position.
RLLM_API int rllm_paged_attention_simt(int dt, const void* q, int q_stride, const void* kcache,
                                       const void* vcache, void* out, int out_stride,
                                       const int* token_seq, const int* positions,
                                       const int* block_table, int bt_stride, int n_tokens, int nh,
                                       int nkv, int hd, int page_size, float scale, int window,
                                       void* stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || hd > MAX_HD || hd % 16 || nkv <= 0 || nh % nkv || page_size <= 0) return ERR_BAD_SIZE;
  if (q_stride % 8 || out_stride % 8) return ERR_BAD_ALIGN;
  const long long warps = (long long)n_tokens * nh;
  const long long blocks = (warps + WARPS - 1) / WARPS;
  if (blocks > 2147483647LL) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  if (dt == DT_F32)
    rc = launch_ex(paged_attention_simt_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, s, 1, 
        (const float*)q, q_stride, (const float*)kcache, (const float*)vcache, (float*)out,
        out_stride, token_seq, positions, block_table, bt_stride, n_tokens, nh, nkv, hd, page_size,
        scale, window);
  else if (dt == DT_BF16)
    rc = launch_ex(paged_attention_simt_kernel<bf16>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, s, 1, 
        (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, (bf16*)out, out_stride,
        token_seq, positions, block_table, bt_stride, n_tokens, nh, nkv, hd, page_size, scale,
        window);
  else return ERR_BAD_DTYPE;
  return rc;
}
