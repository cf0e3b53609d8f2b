// Generic element-wise and row-wise kernels, both precisions: embedding gather,
// RMSNorm, rotary position encoding fused with the write of K and V into the
// paged cache, row gather, residual add, SiLU-gate. All arithmetic in float;
// one rounding on store.
#include "common.cuh"
using namespace rllm;

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :]  (reference: src/gpu/cuda/shaders/embed.cu:24-59)
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int V, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) {           // never read outside the table: flag and emit zeros
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = to_f32(row[i]);
}

RLLM_API int rllm_embed(const int* ids, const void* table, int table_dt, float* out, int T, int H,
                        int V, int* err, void* stream) {
  if (T <= 0) return 0;
  const int threads = H >= 256 ? 256 : (H >= 128 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  if (table_dt == DT_F32) rc = launch_ex(embed_kernel<float>, dim3(T), dim3(threads), 0, s, 1, ids, (const float*)table, out, H, V, err);
  else if (table_dt == DT_BF16) rc = launch_ex(embed_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, ids, (const bf16*)table, out, H, V, err);
  else return ERR_BAD_DTYPE;
  return rc;
}

// ---------------------------------------------------------------- a step's metadata onto the device
// The int32 words of a step's metadata, read straight out of pinned host memory (mapped into the
// device's address space) into the buffer the step's kernels read. The first n_feed words, the
// token ids, come from a device vector instead when one is given: the tokens the step before drew.
// One kernel on the compute stream stands where a host-to-device copy and a device-to-device copy
// would each wait for a copy engine to take over and hand back.
__global__ void step_meta_kernel(const int* __restrict__ host_src, int* __restrict__ dst, int n,
                                 const int* __restrict__ feed, int n_feed) {
  pdl_launch();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    dst[i] = (feed != nullptr && i < n_feed) ? feed[i] : host_src[i];
}

RLLM_API int rllm_step_meta(const int* host_src, int* dst, int n, const int* feed, int n_feed, void* stream) {
  if (n <= 0) return 0;
  const int blocks = (n + 255) / 256 < 32 ? (n + 255) / 256 : 32;
  return launch_ex(step_meta_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 1, host_src, dst, n, feed, n_feed);
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w   (reference: src/gpu/cuda/shaders/rms_norm.cu:78-115)
// x is the float residual stream; w float or bf16; y float or bf16.
// The sum of squares is taken in a fixed order that depends on H only.
// Rows of up to RMS_VEC * 4 * blockDim floats whose length is a multiple of 4 are held in
// registers between the two passes (one read of x); other rows are read twice. Either way the
// order of the sum is the same: thread i takes elements i*4..i*4+3, then (i + blockDim)*4.., a
// tree over the warp, then over the warps.
constexpr int RMS_VEC = 4;

template <typename TW> __device__ __forceinline__ void load4(const TW* p, float (&w)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&w)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&w)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  w[0] = __low2float(a); w[1] = __high2float(a); w[2] = __low2float(b); w[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&a);
  o.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = o;
}

template <typename TW, typename TO, bool VEC>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const TW* __restrict__ w,
                               TO* __restrict__ y, int H, float eps) {
  pdl_launch();
  __shared__ float red[32];
  // rows (when given) come with the step's metadata, which no kernel of the step writes
  const float* xr = x + (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * H;
  TO* yr = y + (size_t)blockIdx.x * H;
  if (VEC) {
    float wv[RMS_VEC][4];
#pragma unroll
    for (int j = 0; j < RMS_VEC; ++j) {                 // weights do not depend on the kernel before
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < H) load4<TW>(w + i, wv[j]);
    }
    pdl_wait();
    float v[RMS_VEC][4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < RMS_VEC; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < H) {
        load4<float>(xr + i, v[j]);
#pragma unroll
        for (int q = 0; q < 4; ++q) ss = fmaf(v[j][q], v[j][q], ss);
      }
    }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < RMS_VEC; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < H) {
        float o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) o[q] = v[j][q] * r * wv[j][q];
        store4(yr + i, o);
      }
    }
  } else {
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_f32<TO>(xr[i] * r * to_f32(w[i]));
  }
}

// Rows whose length is a multiple of 128 * WPR, up to 2,048 * WPR floats: a warp holds a row (WPR = 1) or
// its share of one (2 or 4 warps a row) in registers, 16 bytes a lane and load, all loads of a row in flight
// together, and a CTA of 8 warps takes 8 / WPR rows. The sum is a chain per lane, a tree over the warp and
// then over the row's warps in order: fixed by H alone. One CTA a row (the kernel above) spent most of a
// long portion's norm starting and ending CTAs: 8.8 us for 2,048 rows of 2,048 where the bytes need 4.
template <typename TW, typename TO, int WPR>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                           const TW* __restrict__ w, TO* __restrict__ y, int T, int H,
                                                           float eps) {
  pdl_launch();
  constexpr int RPC = 8 / WPR;                          // rows per CTA
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RPC + warp / WPR, part = warp % WPR;
  const int per = H / WPR;                              // this warp's values: a multiple of 128
  const int n4 = per >> 7;                              // 16-byte loads per lane, at most 16
  const bool live = t < T;
  pdl_wait();
  float4 v[16];
  float ss = 0.f;
  if (live) {
    const float* xr = x + (size_t)(rows ? rows[t] : t) * H + part * per + lane * 4;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < n4) v[j] = __ldcg(reinterpret_cast<const float4*>(xr + j * 128));
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (j < n4) { ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (WPR > 1) {
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < WPR; ++i) ss += red[(warp / WPR) * WPR + i];
  }
  if (!live) return;
  const float r = rsqrtf(ss / (float)H + eps);
  const TW* wr = w + part * per + lane * 4;
  TO* yr = y + (size_t)t * H + part * per + lane * 4;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (j < n4) {
      float wv[4], o[4];
      load4<TW>(wr + j * 128, wv);
      o[0] = v[j].x * r * wv[0]; o[1] = v[j].y * r * wv[1]; o[2] = v[j].z * r * wv[2]; o[3] = v[j].w * r * wv[3];
      store4(yr + j * 128, o);
    }
  }
}

// y[t] = norm(x[rows[t]]) when rows is given, else norm(x[t]).
RLLM_API int rllm_rmsnorm(const float* x, const int* rows, const void* w, int w_dt, void* y, int y_dt, int T,
                          int H, float eps, void* stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  const bool vec = H % 4 == 0 && H <= RMS_VEC * 4 * threads && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)w & 15) == 0 && ((uintptr_t)y & 15) == 0;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  // which kernel takes a row depends on H and the pointers' alignment alone, never on T: a row's sum has the
  // same order whatever step it comes in
  const int wpr = H % 128 == 0 && H <= 2048 ? 1 : (H % 256 == 0 && H <= 4096 ? 2 : (H % 512 == 0 && H <= 8192 ? 4 : 0));
  if (wpr && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)y & 15) == 0) {
    const int rpc = 8 / wpr;
    const dim3 grid((T + rpc - 1) / rpc);
#define ROWS(TW, TO)                                                                                            \
    rc = wpr == 1 ? launch_ex(rmsnorm_rows_kernel<TW, TO, 1>, grid, dim3(256), 0, s, 1, x, rows, (const TW*)w, (TO*)y, T, H, eps) \
       : wpr == 2 ? launch_ex(rmsnorm_rows_kernel<TW, TO, 2>, grid, dim3(256), 0, s, 1, x, rows, (const TW*)w, (TO*)y, T, H, eps) \
                  : launch_ex(rmsnorm_rows_kernel<TW, TO, 4>, grid, dim3(256), 0, s, 1, x, rows, (const TW*)w, (TO*)y, T, H, eps)
    if (w_dt == DT_F32 && y_dt == DT_F32) ROWS(float, float);
    else if (w_dt == DT_F32 && y_dt == DT_BF16) ROWS(float, bf16);
    else if (w_dt == DT_BF16 && y_dt == DT_F32) ROWS(bf16, float);
    else if (w_dt == DT_BF16 && y_dt == DT_BF16) ROWS(bf16, bf16);
    else return ERR_BAD_DTYPE;
#undef ROWS
    return rc;
  }
#define GO(TW, TO)                                                                                              \
  rc = vec ? launch_ex(rmsnorm_kernel<TW, TO, true>, dim3(T), dim3(threads), 0, s, 1, x, rows, (const TW*)w, (TO*)y, H, eps) \
           : launch_ex(rmsnorm_kernel<TW, TO, false>, dim3(T), dim3(threads), 0, s, 1, x, rows, (const TW*)w, (TO*)y, H, eps)
  if (w_dt == DT_F32 && y_dt == DT_F32) GO(float, float);
  else if (w_dt == DT_F32 && y_dt == DT_BF16) GO(float, bf16);
  else if (w_dt == DT_BF16 && y_dt == DT_F32) GO(bf16, float);
  else if (w_dt == DT_BF16 && y_dt == DT_BF16) GO(bf16, bf16);
  else return ERR_BAD_DTYPE;
#undef GO
  return rc;
}

// ---------------------------------------------------------------- RoPE + cache write
// qkv: [T, (nh + 2 nkv) * hd], q heads first, then k heads, then v heads.
// Pair (i, i + rot_dim/2), i < rot_dim/2, of every q and k head is rotated by angle
// pos * inv_freq[i] (float; rot_dim = hd for Llama), q in place; rotated k and plain v go to the paged cache at `slots[t]`
// (= page * page_size + offset, or < 0 to skip the write).
// Cache layout: [page][kv head][offset in page][hd].
// Reference: src/gpu/cuda/shaders/rope.cu:62-77 and attention.cu:295-300.
// The rotation of a step, made once and read by every layer: cs[t][i] = (cos, sin)(positions[t] *
// inv_freq[i]) in float, i < n_freq. The same sincosf the kernels below call when they get no table.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int T, int n_freq) {
  pdl_launch();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * n_freq) return;
  const int t = idx / n_freq, i = idx % n_freq;
  float sn, c;
  sincosf((float)positions[t] * inv_freq[i], &sn, &c);
  cs[idx] = make_float2(c, sn);
}
RLLM_API int rllm_rope_table(const int* positions, const float* inv_freq, void* cs, int T, int n_freq,
                             void* stream) {
  if (T <= 0 || n_freq <= 0) return 0;
  const int n = T * n_freq;
  return launch_ex(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, 1, positions,
                   inv_freq, (float2*)cs, T, n_freq);
}

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, const float2* __restrict__ cos_sin,
                                  const int* __restrict__ slots,
                                  T* __restrict__ kcache, T* __restrict__ vcache, int nh, int nkv,
                                  int hd, int page_size, int rot_dim) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = hd / 2;
  const int width = (nh + 2 * nkv) * hd;
  T* row = qkv + (size_t)t * width;
  const float pos = (float)positions[t];
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int rh = rot_dim / 2;                 // rotated pairs are (i, i + rh), i < rh
  const int n_rot = (nh + nkv) * half;
  for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
    const int head = idx / half, i = idx % half;
    T* hp = row + (size_t)head * hd;
    int ia, ib;
    if (i < rh) { ia = i; ib = i + rh; } else { ia = rot_dim + 2 * (i - rh); ib = ia + 1; }
    float a = to_f32(hp[ia]), b = to_f32(hp[ib]);
    float ra = a, rb = b;
    if (i < rh) {
      float sn, cs;
      if (cos_sin) { const float2 v = cos_sin[(size_t)t * rh + i]; cs = v.x; sn = v.y; }
      else sincosf(pos * inv_freq[i], &sn, &cs);
      ra = a * cs - b * sn;
      rb = a * sn + b * cs;
    }
    if (head < nh) {
      if (i < rh) { hp[ia] = from_f32<T>(ra); hp[ib] = from_f32<T>(rb); }
    } else if (slot >= 0) {
      const int kvh = head - nh;
      T* dst = kcache + (((size_t)page * nkv + kvh) * page_size + off) * hd;
      dst[ia] = from_f32<T>(ra);
      dst[ib] = from_f32<T>(rb);
    }
  }
  if (slot >= 0) {
    const T* vrow = row + (size_t)(nh + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
      const int kvh = idx / hd, d = idx % hd;
      vcache[(((size_t)page * nkv + kvh) * page_size + off) * hd + d] = vrow[idx];
    }
  }
}

// The same for bfloat16 with whole heads rotated (rot_dim == hd, hd a multiple of 16) and the
// step's table of angles: eight pairs per thread, 16-byte loads and stores.
__global__ void rope_cache_vec_kernel(bf16* __restrict__ qkv, const float2* __restrict__ cos_sin,
                                      const int* __restrict__ slots, bf16* __restrict__ kcache,
                                      bf16* __restrict__ vcache, int nh, int nkv, int hd, int page_size) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = hd / 2, cph = half / 8;             // chunks of eight pairs per head
  bf16* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const float2* cs_row = cos_sin + (size_t)t * half;
  for (int idx = threadIdx.x; idx < (nh + nkv) * cph; idx += blockDim.x) {
    const int head = idx / cph, c = idx % cph;
    bf16* hp = row + (size_t)head * hd + 8 * c;
    const uint4 ra = *reinterpret_cast<const uint4*>(hp), rb = *reinterpret_cast<const uint4*>(hp + half);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&rb);
    const float4* cs4 = reinterpret_cast<const float4*>(cs_row + 8 * c);     // (cos, sin) pairs, two per float4
    uint4 oa, ob;
    uint32_t* oa32 = reinterpret_cast<uint32_t*>(&oa);
    uint32_t* ob32 = reinterpret_cast<uint32_t*>(&ob);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 cs = cs4[e];                         // pair 2e: (x, y), pair 2e + 1: (z, w)
      const float a0 = __low2float(a2[e]), a1 = __high2float(a2[e]);
      const float b0 = __low2float(b2[e]), b1 = __high2float(b2[e]);
      const __nv_bfloat162 na = __floats2bfloat162_rn(a0 * cs.x - b0 * cs.y, a1 * cs.z - b1 * cs.w);
      const __nv_bfloat162 nb = __floats2bfloat162_rn(a0 * cs.y + b0 * cs.x, a1 * cs.w + b1 * cs.z);
      oa32[e] = *reinterpret_cast<const uint32_t*>(&na);
      ob32[e] = *reinterpret_cast<const uint32_t*>(&nb);
    }
    if (head < nh) {
      *reinterpret_cast<uint4*>(hp) = oa;
      *reinterpret_cast<uint4*>(hp + half) = ob;
    } else if (slot >= 0) {
      bf16* dst = kcache + (((size_t)page * nkv + (head - nh)) * page_size + off) * hd + 8 * c;
      *reinterpret_cast<uint4*>(dst) = oa;
      *reinterpret_cast<uint4*>(dst + half) = ob;
    }
  }
  if (slot >= 0) {
    const bf16* vrow = row + (size_t)(nh + nkv) * hd;
    const int vph = hd / 8;
    for (int idx = threadIdx.x; idx < nkv * vph; idx += blockDim.x) {
      const int kvh = idx / vph, c = idx % vph;
      *reinterpret_cast<uint4*>(vcache + (((size_t)page * nkv + kvh) * page_size + off) * hd + 8 * c) =
          *reinterpret_cast<const uint4*>(vrow + (size_t)kvh * hd + 8 * c);
    }
  }
}

// cos_sin: the table of rllm_rope_table for these positions ([T][rot_dim / 2] float2), or null.
RLLM_API int rllm_rope_cache_write(void* qkv, int dt, const int* positions, const float* inv_freq,
                                   const void* cos_sin, const int* slots, void* kcache, void* vcache, int T, int nh,
                                   int nkv, int hd, int page_size, int rot_dim, void* stream) {
  if (T <= 0) return 0;
  if (hd % 2 || rot_dim % 2 || rot_dim > hd || rot_dim < 0) return ERR_BAD_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  const int work = (nh + nkv) * hd / 2;
  const int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)cos_sin) & 15) == 0 &&
                       (!slots || (((uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0);
  if (dt == DT_BF16 && cos_sin && rot_dim == hd && hd % 16 == 0 && aligned)
    return launch_ex(rope_cache_vec_kernel, dim3(T), dim3(128), 0, s, 1, (bf16*)qkv, (const float2*)cos_sin, slots,
                     (bf16*)kcache, (bf16*)vcache, nh, nkv, hd, page_size);
  if (dt == DT_F32)
    rc = launch_ex(rope_cache_kernel<float>, dim3(T), dim3(threads), 0, s, 1, (float*)qkv, positions, inv_freq, (const float2*)cos_sin, slots,
                                                   (float*)kcache, (float*)vcache, nh, nkv, hd,
                                                   page_size, rot_dim);
  else if (dt == DT_BF16)
    rc = launch_ex(rope_cache_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, (bf16*)qkv, positions, inv_freq, (const float2*)cos_sin, slots,
                                                  (bf16*)kcache, (bf16*)vcache, nh, nkv, hd,
                                                  page_size, rot_dim);
  else return ERR_BAD_DTYPE;
  return rc;
}

// ---------------------------------------------------------------- small helpers
// out[r, :] = x[rows[r], :]   (float rows of the residual stream)
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int H) {
  pdl_launch();
  pdl_wait();
  const float* src = x + (size_t)rows[blockIdx.x] * H;
  float* dst = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}
RLLM_API int rllm_gather_rows(const float* x, const int* rows, float* out, int R, int H, void* stream) {
  if (R <= 0) return 0;
  int rc = launch_ex(gather_rows_kernel, dim3(R), dim3(H >= 256 ? 256 : 64), 0, (cudaStream_t)stream, 1, x, rows, out, H);
  return rc;
}

// residual[i] += delta[i]   (float accumulate; delta float or bf16)
template <typename T>
__global__ void add_into_kernel(float* __restrict__ res, const T* __restrict__ delta, size_t n) {
  pdl_launch();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) res[i] += to_f32(delta[i]);
}
RLLM_API int rllm_add_into(float* res, const void* delta, int dt, long long n, void* stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  if (dt == DT_F32) rc = launch_ex(add_into_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, res, (const float*)delta, (size_t)n);
  else if (dt == DT_BF16) rc = launch_ex(add_into_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, res, (const bf16*)delta, (size_t)n);
  else return ERR_BAD_DTYPE;
  return rc;
}

// y[t, n] += bias[n] in place, the sum formed in float (y and bias of one type, float or bf16):
// the bias of a projection whose product ran without one (src/model/primitives.rs:60-83 adds it
// the same way, after the product).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const T* __restrict__ bias, int rows, int N, long long ld) {
  pdl_launch();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * N) return;
  const int n = (int)(i % N);
  T* p = y + (size_t)(i / N) * ld + n;
  *p = from_f32<T>(to_f32(*p) + to_f32(bias[n]));
}
RLLM_API int rllm_add_bias(void* y, const void* bias, int dt, int rows, int N, long long ld, void* stream) {
  if (rows <= 0 || N <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)(((size_t)rows * N + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32) return launch_ex(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (float*)y, (const float*)bias, rows, N, ld);
  if (dt == DT_BF16) return launch_ex(add_bias_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (bf16*)y, (const bf16*)bias, rows, N, ld);
  return ERR_BAD_DTYPE;
}

// Checked runs: a step's block tables and cache slots are tested before any kernel uses them. An
// entry outside [-1, num_pages) of a table, or a slot outside [-1, num_pages * page_size), is put to
// -1, which every kernel reads as "no page here" / "do not write", so the access is skipped instead
// of made; the error word gets 1 + the index of the first offender (first failure wins). This
// stands in for a memory checker: a wrong table shows as an error naming the entry, not as a fault
// or as silently wrong logits. (The reference checks its handles on the host only:
// src/model/kv_cache.rs:864-875.)
__global__ void check_meta_kernel(int* __restrict__ block_table, int n_table, int* __restrict__ slots, int n_slots,
                                  int num_pages, int page_size, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_table) {
    const int v = block_table[i];
    if (v < -1 || v >= num_pages) { block_table[i] = -1; atomicCAS(err, 0, 1 + i); }
  } else if (i - n_table < n_slots) {
    const int j = i - n_table, v = slots[j];
    if (v < -1 || (long long)v >= (long long)num_pages * page_size) { slots[j] = -1; atomicCAS(err, 0, 0x40000000 | j); }
  }
}
RLLM_API int rllm_check_meta(int* block_table, int n_table, int* slots, int n_slots, int num_pages, int page_size,
                             int* err, void* stream) {
  if (!err || num_pages < 0 || page_size <= 0) return ERR_BAD_SIZE;
  const int n = (block_table ? n_table : 0) + (slots ? n_slots : 0);
  if (n <= 0) return 0;
  return launch_ex(check_meta_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, 1, block_table,
                   block_table ? n_table : 0, slots, slots ? n_slots : 0, num_pages, page_size, err);
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i]   (reference: elementwise.cu:36-49)
template <typename T>
__global__ void silu_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t n) {
  pdl_launch();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  size_t t = idx / I; int i = (int)(idx % I);
  float g = to_f32(gu[t * 2 * I + i]), u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
}
RLLM_API int rllm_silu_gate(const void* gu, void* out, int dt, int T, int I, void* stream) {
  size_t n = (size_t)T * I;
  if (n == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  if (dt == DT_F32) rc = launch_ex(silu_gate_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, I, n);
  else if (dt == DT_BF16) rc = launch_ex(silu_gate_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu, (bf16*)out, I, n);
  else return ERR_BAD_DTYPE;
  return rc;
}
