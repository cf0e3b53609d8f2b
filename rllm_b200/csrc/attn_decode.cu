// Decode attention over the paged bfloat16 cache: every sequence brings ONE query token.
//
// The work is pure memory traffic (each key and value is read once and used by the G query
// heads of its kv head), so the kernel is built around keeping bytes in flight:
//   * a CTA serves one (sequence, kv head, range of keys); the ranges of a sequence form a
//     thread-block cluster along z;
//   * one producer warp walks the block table and issues TMA tensor copies, two per page
//     (keys, values), 128-byte swizzled, into a ring of tiles of 64 keys (32 for head size 128); an mbarrier
//     per stage counts the bytes;
//   * four consumer warps take the tiles round-robin. Each holds the G query rows as the
//     A operand of mma.sync m16n8k16 (rows beyond G are zero), computes scores, the running
//     maximum/sum softmax in float with exp2, and the weighted sum of values, all from the
//     swizzled tile with ldmatrix;
//   * the four warps' partial results are merged in shared memory, then the ranges of the
//     cluster are merged through distributed shared memory in rank order, and the output row is
//     written once. No scratch memory in global memory, no second kernel.
// A key j is visible when j <= pos (pos = kv_len - 1) and j > pos - window if a window is set.
// Pages the table does not hold (given back by a window, or beyond the sequence in the last
// tile) are replaced by the page of `pos`, whose contents are finite; their keys are masked.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:328-388 of the reference (scale, softmax with
// the maximum subtracted, weighted V, head h -> kv head h / G, window start :337-338).
// Cache layout: [page][kv head][offset in page][HD]; page_size 8, 16, 32 or 64 and at most a tile
// (64 keys for HD 64, 32 keys for HD 128).
//
// Programmatic dependent launch: tiles that cannot hold the token the previous kernel has just
// written are fetched before the wait for that kernel.
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>
#include <unordered_map>

using namespace rllm;
using namespace sm100;

namespace {

constexpr int NW = 4;                    // consumer warps
constexpr int THREADS = (NW + 1) * 32;   // + one producer warp
constexpr int MAX_CLUSTER = 8;

struct DecParams {
  const bf16* q; int q_stride;
  bf16* out; int out_stride;
  const int* kv_lens; const int* block_table; int bt_stride;
  int nh, nkv, page_size, window, splits;
  float scale_log2e;
  int* err;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `ch` of key row `r` inside a K or V tile: 64-column sub-tiles
// of [TILE rows][128 bytes], chunk index XORed with the row (the TMA 128-byte swizzle).
template <int TILE>
__device__ __forceinline__ uint32_t tile_off(int r, int ch) {
  return (uint32_t)((ch >> 3) * (TILE * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
}

template <int HD> struct DCfg {
  static constexpr int TILE = 4096 / HD;                      // keys per stage: 64 (HD 64), 32 (HD 128)
  static constexpr int KV_BYTES = TILE * HD * 2;              // one K (or V) tile: 8 KB
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  // A stage is always consumed by the same warp (STAGES is a multiple of NW and tile i goes to
  // warp i % NW, stage i % STAGES), so no warp can ask for a later use of a stage before it has
  // itself consumed the earlier one.
  static constexpr int STAGES = NW;                           // 64 KB in flight per CTA, 3 CTAs per SM
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // after the ring: per-warp partial results [NW][G][HD], their (max, sum) [NW][16] each, then the
  // CTA's merged partial [G][HD] and its (max, sum) [16] each, all float
  static constexpr int merge_floats(int G) { return NW * G * HD + 2 * NW * 16 + G * HD + 32; }
  static constexpr int smem_bytes(int G) { return 1024 + RING_BYTES + merge_floats(G) * 4; }
};

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const DecParams p) {
  typedef DCfg<HD> C;
  constexpr int TILE = C::TILE;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  static_assert(C::STAGES % NW == 0, "a stage must always belong to the same consumer warp");
  extern __shared__ uint8_t dsmem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[C::STAGES];
  __shared__ int abort_flag;
  __shared__ int never_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)dsmem_raw + 1023) & ~(uintptr_t)1023);
  const int kvh = blockIdx.x, seq = blockIdx.y;
  const int rank = p.splits > 1 ? (int)cluster_rank() : 0;
  const int G = p.nh / p.nkv;
  // merge areas: per warp, then per CTA (the latter is read by the other ranks of the cluster)
  float* w_o = reinterpret_cast<float*>(smem + C::RING_BYTES);     // [NW][G][HD]
  float* w_m = w_o + NW * G * HD;                                  // [NW][16]
  float* w_l = w_m + NW * 16;                                      // [NW][16]
  float* c_o = w_l + NW * 16;                                      // [G][HD]
  float* c_m = c_o + G * HD;                                       // [16]
  float* c_l = c_m + 16;                                           // [16]

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    abort_flag = 0;
    never_flag = 0;
    fence_barrier_init();
  }
  if (warp == NW && lane == 0) { prefetch_tensormap(&tmap_k); prefetch_tensormap(&tmap_v); }
  __syncthreads();
  pdl_launch();

  // kv_lens and the block table come from the host copy that precedes the whole step, not from
  // the kernel before this one, so they may be read before the wait
  const int kv_len = p.kv_lens[seq];
  const int pos = kv_len - 1;
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int tile_first = lo / TILE;
  const int tiles_total = pos / TILE + 1 - tile_first;
  const int per = (tiles_total + p.splits - 1) / p.splits;
  const int tb = tile_first + rank * per;
  const int te = min(tile_first + tiles_total, tb + per);
  const int n_tiles = te > tb ? te - tb : 0;
  const int last_tile = pos / TILE;                         // the tile the newest token lies in

  if (warp == NW) {
    // ------------------------------------------------------------ producer
    const int ppt = TILE / p.page_size;                     // pages per tile
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;
    const int pos_page = bt[pos / p.page_size];
    const int last_held = pos / p.page_size;
    bool waited = false, ok = true;
    int issued = 0;
    for (int i0 = 0; i0 < n_tiles && ok; i0 += 32 / ppt) {
      // the page ids of up to 32 pages (32 / ppt tiles) in one load
      const int pg_idx = (tb + i0) * ppt + lane;
      int page = (pg_idx <= last_held) ? bt[pg_idx] : -1;
      if (page < 0) page = pos_page;
      const int n_here = min(32 / ppt, n_tiles - i0);
      for (int ii = 0; ii < n_here && ok; ++ii) {
        const int i = i0 + ii;
        const int s = i % C::STAGES;
        const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
        if (tb + i == last_tile && !waited) { pdl_wait(); waited = true; }
        if (lane == 0) {
          if (i >= C::STAGES && !mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag)) {
            abort_flag = 1; record_failure(p.err, 11, (i & 0xfff) | (seq << 12)); ok = false;
          }
          if (ok) mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        uint8_t* st = smem + (size_t)s * C::STAGE_BYTES;
        for (int j = 0; j < ppt; ++j) {
          const int pj = __shfl_sync(0xffffffffu, page, ii * ppt + j);
          if (lane == 0) {
            const int row = (pj * p.nkv + kvh) * p.page_size;
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) {
              tma_load_2d(st + h * (TILE * 128) + j * p.page_size * 128, &tmap_k, &full_bar[s], h * 64, row);
              tma_load_2d(st + C::KV_BYTES + h * (TILE * 128) + j * p.page_size * 128, &tmap_v, &full_bar[s],
                          h * 64, row);
            }
          }
        }
        issued = i + 1;
      }
    }
    if (!waited) pdl_wait();
    if (lane == 0 && abort_flag) {
      for (int i = max(0, issued - C::STAGES); i < issued; ++i)
        mbar_wait(&full_bar[i % C::STAGES], (uint32_t)(i / C::STAGES) & 1u, &never_flag, 200000000LL);
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int quad = lane >> 2, qi = lane & 3;
    const bool vA = quad < G, vB = quad + 8 < G;
    pdl_wait();                                   // q comes from the kernel before this one
    uint32_t qf[KSTEPS][4];
    {
      const bf16* qa = p.q + (size_t)seq * p.q_stride + (size_t)(kvh * G + (vA ? quad : 0)) * HD;
      const bf16* qb = p.q + (size_t)seq * p.q_stride + (size_t)(kvh * G + (vB ? quad + 8 : 0)) * HD;
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
    const int mat = lane >> 3, rr = lane & 7;
    bool ok = true;

    for (int i = warp; i < n_tiles && ok; i += NW) {
      const int s = i % C::STAGES;
      const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
      bool got = true;
      if (lane == 0) got = mbar_wait(&full_bar[s], ph, &abort_flag);
      got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
      if (!got) { if (lane == 0) { abort_flag = 1; record_failure(p.err, 12, (i & 0xfff) | (seq << 12)); } ok = false; break; }
      const uint32_t kt = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
      const uint32_t vt = kt + C::KV_BYTES;
      const int j0 = (tb + i) * TILE;

      float sc[TILE / 8][4];
#pragma unroll
      for (int x = 0; x < TILE / 8; ++x) { sc[x][0] = sc[x][1] = sc[x][2] = sc[x][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int nt = 0; nt < TILE / 8; nt += 2) {
          uint32_t b[4];
          ldsm_x4(b, kt + tile_off<TILE>((nt + (mat >> 1)) * 8 + rr, 2 * kk + (mat & 1)));
          mma16816(sc[nt], qf[kk], b[0], b[1]);
          mma16816(sc[nt + 1], qf[kk], b[2], b[3]);
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < TILE / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j0 + nt * 8 + qi * 2 + e;
          const bool vis = j <= pos && j >= lo;
          sc[nt][e] = (vis && vA) ? sc[nt][e] * p.scale_log2e : -INFINITY;
          sc[nt][2 + e] = (vis && vB) ? sc[nt][2 + e] * p.scale_log2e : -INFINITY;
          mxA = fmaxf(mxA, sc[nt][e]);
          mxB = fmaxf(mxB, sc[nt][2 + e]);
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
      const float useA = (mnA == -INFINITY) ? 0.f : mnA, useB = (mnB == -INFINITY) ? 0.f : mnB;
      const float corrA = exp2f(mA - useA), corrB = exp2f(mB - useB);     // exp2(-inf) = 0
      mA = mnA; mB = mnB;
      lA *= corrA; lB *= corrB;
#pragma unroll
      for (int x = 0; x < DTILES; ++x) { o[x][0] *= corrA; o[x][1] *= corrA; o[x][2] *= corrB; o[x][3] *= corrB; }
#pragma unroll
      for (int kb = 0; kb < TILE / 16; ++kb) {
        uint32_t a[4];
        {
          const float p0 = exp2f(sc[2 * kb][0] - useA), p1 = exp2f(sc[2 * kb][1] - useA);
          const float p2 = exp2f(sc[2 * kb][2] - useB), p3 = exp2f(sc[2 * kb][3] - useB);
          const float p4 = exp2f(sc[2 * kb + 1][0] - useA), p5 = exp2f(sc[2 * kb + 1][1] - useA);
          const float p6 = exp2f(sc[2 * kb + 1][2] - useB), p7 = exp2f(sc[2 * kb + 1][3] - useB);
          lA += p0 + p1 + p4 + p5;
          lB += p2 + p3 + p6 + p7;
          a[0] = pack2(p0, p1); a[1] = pack2(p2, p3);
          a[2] = pack2(p4, p5); a[3] = pack2(p6, p7);
        }
#pragma unroll
        for (int dn = 0; dn < DTILES; dn += 2) {
          uint32_t b[4];
          ldsm_x4_t(b, vt + tile_off<TILE>(kb * 16 + (mat & 1) * 8 + rr, dn + (mat >> 1)));
          mma16816(o[dn], a, b[0], b[1]);
          mma16816(o[dn + 1], a, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);       // the stage may be refilled
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    // park this warp's partial result (rows beyond G hold zeros and -inf)
#pragma unroll
    for (int dn = 0; dn < DTILES; ++dn) {
      const int d = dn * 8 + qi * 2;
      if (vA) *reinterpret_cast<float2*>(w_o + ((size_t)warp * G + quad) * HD + d) = make_float2(o[dn][0], o[dn][1]);
      if (vB) *reinterpret_cast<float2*>(w_o + ((size_t)warp * G + quad + 8) * HD + d) = make_float2(o[dn][2], o[dn][3]);
    }
    if (qi == 0) {
      w_m[warp * 16 + quad] = mA; w_l[warp * 16 + quad] = lA;
      w_m[warp * 16 + quad + 8] = mB; w_l[warp * 16 + quad + 8] = lB;
    }
  }
  __syncthreads();

  // ---------------------------------------------------------------- merge the four warps
  for (int idx = threadIdx.x; idx < G * HD; idx += THREADS) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, w_m[w * 16 + r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float f = (w_m[w * 16 + r] == -INFINITY) ? 0.f : exp2f(w_m[w * 16 + r] - M);
      L += w_l[w * 16 + r] * f;
      O += w_o[((size_t)w * G + r) * HD + d] * f;
    }
    if (p.splits == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      p.out[(size_t)seq * p.out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(O * inv);
    } else {
      c_o[r * HD + d] = O;
      if (d == 0) { c_m[r] = M; c_l[r] = L; }
    }
  }
  if (p.splits > 1) {
    // ---------------------------------------------------------------- merge the ranges of the cluster
    __syncwarp();
    cluster_sync_all();
    if (!abort_flag) {
      uint32_t bo[MAX_CLUSTER], bm[MAX_CLUSTER], bl[MAX_CLUSTER];
#pragma unroll
      for (int s = 0; s < MAX_CLUSTER; ++s) {
        const uint32_t rk = s < p.splits ? (uint32_t)s : 0u;
        bo[s] = map_to_rank(smem_u32(c_o), rk);
        bm[s] = map_to_rank(smem_u32(c_m), rk);
        bl[s] = map_to_rank(smem_u32(c_l), rk);
      }
      // row r is finished by rank r % splits
      for (int idx = threadIdx.x; idx < G * HD; idx += THREADS) {
        const int r = idx / HD, d = idx % HD;
        if (r % p.splits != rank) continue;
        float ms[MAX_CLUSTER];
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
          ms[s] = s < p.splits ? ld_cluster_f32(bm[s] + (uint32_t)r * 4) : -INFINITY;
          M = fmaxf(M, ms[s]);
        }
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
          if (s < p.splits && ms[s] != -INFINITY) {
            const float f = exp2f(ms[s] - M);
            L += ld_cluster_f32(bl[s] + (uint32_t)r * 4) * f;
            O += ld_cluster_f32(bo[s] + (uint32_t)(r * HD + d) * 4) * f;
          }
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        p.out[(size_t)seq * p.out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(O * inv);
      }
    }
    __syncwarp();
    cluster_sync_all();          // nobody leaves while its shared memory is still read
  }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_enc = nullptr;
std::mutex g_dmu;

int get_enc() {
  if (g_enc) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return -5;
  }
  g_enc = (EncodeTiledFn)fn;
  return 0;
}

struct CKey {
  const void* p; long long rows; int hd, box;
  bool operator==(const CKey& o) const { return p == o.p && rows == o.rows && hd == o.hd && box == o.box; }
};
struct CHash {
  size_t operator()(const CKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows * 31 + k.hd) << 1) ^ (size_t)k.box;
  }
};
std::unordered_map<CKey, CUtensorMap, CHash> g_cache_maps;     // one per cache tensor, kept for the process

// the cache as a matrix [pages * nkv * page_size, hd]; box = 64 columns x page_size rows
int cache_map(CUtensorMap* out, const void* ptr, long long rows, int hd, int page_size) {
  std::lock_guard<std::mutex> lk(g_dmu);
  CKey key{ptr, rows, hd, page_size};
  auto it = g_cache_maps.find(key);
  if (it == g_cache_maps.end()) {
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)page_size};
    cuuint32_t estr[2] = {1, 1};
    if (g_enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -5;
    if (g_cache_maps.size() > 1024) g_cache_maps.clear();
    it = g_cache_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

template <int HD>
int launch_dec(const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, int num_seqs, cudaStream_t s) {
  typedef DCfg<HD> C;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::smem_bytes(16)) != cudaSuccess) { cudaGetLastError(); return -5; }
    configured = true;
  }
  dim3 grid(p.nkv, num_seqs, p.splits);
  if (grid.y > 65535) return ERR_TOO_LARGE;
  return launch_ex(attn_decode_kernel<HD>, grid, dim3(THREADS), C::smem_bytes(p.nh / p.nkv), s, p.splits, mk, mv, p);
}

}  // namespace

// q: [S, ...] bf16, one row per sequence, stride q_stride, head h at h*hd; out likewise.
// kcache / vcache: [num_pages][nkv][page_size][hd] bf16. kv_lens [S]: keys visible to each
// sequence's token (its own included). splits: ranges of keys per sequence (1..8, one cluster).
RLLM_API int rllm_attention_decode(const void* q, int q_stride, const void* kcache, const void* vcache,
                                   long long num_pages, void* out, int out_stride, const int* kv_lens,
                                   const int* block_table, int bt_stride, int num_seqs, int nh, int nkv, int hd,
                                   int page_size, float scale, int window, int splits, int* err, void* stream) {
  if (num_seqs <= 0) return 0;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || nh / nkv > 16) return ERR_BAD_SIZE;
  if ((page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) || page_size > 4096 / hd)
    return ERR_BAD_SIZE;                          // a page must fit in one tile of 4096 / hd keys
  if (splits < 1 || splits > MAX_CLUSTER || num_pages <= 0) return ERR_BAD_SIZE;
  if (q_stride % 2 || out_stride % 2 || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) ||
      ((uintptr_t)kcache & 127) || ((uintptr_t)vcache & 127)) return ERR_BAD_ALIGN;
  int rc = get_enc();
  if (rc) return rc;
  CUtensorMap mk, mv;
  const long long rows = num_pages * nkv * page_size;
  if ((rc = cache_map(&mk, kcache, rows, hd, page_size))) return rc;
  if ((rc = cache_map(&mv, vcache, rows, hd, page_size))) return rc;
  DecParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
  p.kv_lens = kv_lens; p.block_table = block_table; p.bt_stride = bt_stride; p.nh = nh; p.nkv = nkv;
  p.page_size = page_size; p.window = window; p.splits = splits; p.scale_log2e = scale * 1.4426950408889634f;
  p.err = err;
  cudaStream_t s = (cudaStream_t)stream;
  return hd == 64 ? launch_dec<64>(mk, mv, p, num_seqs, s) : launch_dec<128>(mk, mv, p, num_seqs, s);
}
