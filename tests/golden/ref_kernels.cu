// Host launchers around the reference project's own CUDA kernels, unmodified: each section
// #includes one shader file of JonCooperWorks/rLLM (src/gpu/cuda/shaders/) and adds a plain C
// function that fills the kernel's parameter block and launches it. The shader files define the
// same helper names, so this file is compiled once per shader with -DWRAP_<NAME> and
// -I<reference>/src/gpu/cuda/shaders; `make_golden.py` does that and calls the launchers through
// ctypes. Launch shapes follow the kernels' own index arithmetic (every kernel guards its range).
// Nothing here is part of the engine; it exists to produce the golden logits beside it.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#define API extern "C" __attribute__((visibility("default")))
typedef __nv_bfloat16 bf;

#if defined(WRAP_EMBED)
#include "embed.cu"
API void ref_embed(unsigned token, unsigned hidden, const bf* table, bf* out) {
  EmbedParams p; p.token_id = token; p.hidden_dim = hidden;
  embed_lookup<<<(hidden + 255) / 256, 256>>>(p, table, out);
}
#elif defined(WRAP_RMS_NORM)
#include "rms_norm.cu"
API void ref_rms_norm(unsigned hidden, float eps, const bf* in, const bf* w, bf* out) {
  RmsNormParams p; p.hidden_size = hidden; p.eps = eps;
  rms_norm<<<1, 256>>>(p, in, w, out);
}
#elif defined(WRAP_MATMUL)
#include "matmul.cu"
API void ref_matvec(unsigned M, unsigned K, const bf* W, const bf* x, bf* y) {
  MatvecParams p; p.M = M; p.K = K;
  matvec_bf16<<<(M * 32 + 255) / 256, 256>>>(p, W, x, y);
}
#elif defined(WRAP_ROPE)
#include "rope.cu"
API void ref_rope(unsigned pos, float theta, unsigned nh, unsigned nkv, unsigned hd, bf* q, bf* k) {
  RopeParams p; p.pos = pos; p.rope_theta = theta; p.num_heads = nh; p.num_kv_heads = nkv; p.head_dim = hd;
  const unsigned pairs = (nh + nkv) * (hd / 2);
  rotary_embedding<<<(pairs + 255) / 256, 256>>>(p, q, k);
}
#elif defined(WRAP_ATTENTION)
#include "attention.cu"
API void ref_copy_kv(unsigned pos, unsigned nkv, unsigned hd, const bf* src, bf* cache) {
  CopyKvParams p; p.pos = pos; p.num_kv_heads = nkv; p.head_dim = hd;
  copy_to_kv_cache<<<(nkv * hd + 255) / 256, 256>>>(p, src, cache);
}
API void ref_attention(unsigned seq_len, unsigned nh, unsigned nkv, unsigned hd, unsigned window, const bf* q,
                       const bf* kc, const bf* vc, bf* out) {
  AttentionParams p; p.seq_len = seq_len; p.num_heads = nh; p.num_kv_heads = nkv; p.head_dim = hd;
  p.window_size = window; p.attn_scale = 0.0f;                   // 0: the kernel's own head_dim^-1/2
  attention<<<nh, 256>>>(p, q, kc, vc, out);
}
#elif defined(WRAP_ELEMENTWISE)
#include "elementwise.cu"
API void ref_silu_mul(unsigned n, const bf* gate, const bf* up, bf* out) {
  ElemParams p; p.size = n;
  silu_mul<<<(n + 255) / 256, 256>>>(p, gate, up, out);
}
API void ref_add(unsigned n, const bf* a, const bf* b, bf* out) {
  ElemParams p; p.size = n;
  add_tensors<<<(n + 255) / 256, 256>>>(p, a, b, out);
}
API int ref_sync() { return (int)cudaDeviceSynchronize(); }
#endif
