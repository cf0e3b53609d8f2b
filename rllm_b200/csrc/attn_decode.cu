// Decode attention over the paged bfloat16 cache: every sequence brings ONE query token.
//
// The work is pure memory traffic (each key and value is read once and used by the G query
// heads of its kv head), so the kernel is built around keeping bytes in flight:
//   * a CTA serves one (sequence, kv head, range of keys); the ranges of a sequence form a
//     thread-block cluster along z;
//   * every warp fetches its own tiles (tile i of the range goes to warp i % NW) with 16-byte
//     asynchronous copies (cp.async), each lane looking up the page of its key row in the block
//     table, into stages of its own, written in the 128-byte swizzled layout that ldmatrix reads
//     without bank conflicts. D tiles per warp are on the way while it works on one. (Tensor
//     copies by TMA, one per page, topped out at two thirds of the memory bandwidth here: a
//     page of 16 positions is 2 KB per kv head, too small a box for the copy engine.)
//   * the warp holds the G query rows as the A operand of mma.sync m16n8k16 (rows beyond G are
//     zero), computes scores, the running maximum/sum softmax in float with exp2, and the
//     weighted sum of values;
//   * the warps' partial results are merged in shared memory, then the ranges of the cluster
//     are merged through distributed shared memory in rank order, and the output row is
//     written once. No scratch memory in global memory, no second kernel.
// A key j is visible when j <= pos (pos = kv_len - 1) and j > pos - window if a window is set.
// Pages the table does not hold (given back by a window, or beyond the sequence in the last
// tile) are replaced by the page of `pos`, whose contents are finite; their keys are masked.
//
// Formulas: src/gpu/cuda/shaders/attention.cu:328-388 of the reference (scale, softmax with
// the maximum subtracted, weighted V, head h -> kv head h / G, window start :337-338).
// Cache layout: [page][kv head][offset in page][HD]; any page size.
//
// Programmatic dependent launch: tiles that cannot hold the token the previous kernel has just
// written are fetched before the wait for that kernel.
#include "common.cuh"
#include "sm100.cuh"

using namespace rllm;
using namespace sm100;

namespace {

// Warps per CTA and tiles in flight per warp, per head size. Two CTAs share an SM; the time of a
// tile is a chain of dependent steps inside its warp (fragments, products, softmax), so warps
// count for more than depth: at head size 64 six warps with two tiles each in flight beat four
// with three (batch 8 x 4,096 keys: 15.1 against 16.1 us, batch 64: 86 against 96 us). At head
// size 128 the kernel needs 186 registers a thread, and six warps would leave one CTA per SM.
// warps per CTA and tiles in flight per warp, by head size (measured: six warps with two tiles each
// beat four with three at head size 64; eight need a whole SM and lose), and the tile's size
constexpr int ADEC_NW = 6, ADEC_D = 2;           // head size 64
constexpr int ADEC_NW128 = 4, ADEC_D128 = 3;     // head size 128
constexpr int ADEC_TILE_KB = 4;                  // K (and V) bytes per tile, in KB
constexpr int MAX_CLUSTER = 16;       // ranges of a sequence's keys; more than 8 CTAs in a cluster need the kernel's own permission

struct DecParams {
  const bf16* q; int q_stride;
  const bf16* kcache; const bf16* vcache;
  bf16* out; int out_stride;
  const int* kv_lens; const int* block_table; int bt_stride;
  int nh, nkv, page_size, window, splits;
  int page_shift;       // log2(page_size), or -1 when it is no power of two
  float scale_log2e;
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
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {          // exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `ch` of key row `r` inside a K or V tile: 64-column sub-tiles
// of [TILE rows][128 bytes], chunk index XORed with the row (the 128-byte swizzle).
template <int TILE>
__device__ __forceinline__ uint32_t tile_off(int r, int ch) {
  return (uint32_t)((ch >> 3) * (TILE * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
}

template <int HD> struct DCfg {
  static constexpr int NW = HD == 64 ? ADEC_NW : ADEC_NW128;  // warps per CTA
  static constexpr int D = HD == 64 ? ADEC_D : ADEC_D128;     // tiles in flight per warp
  static constexpr int THREADS = NW * 32;
  static constexpr int KV_BYTES = ADEC_TILE_KB * 1024;        // one K (or V) tile
  static constexpr int TILE = KV_BYTES / (HD * 2);            // keys per tile: 32 (HD 64), 16 (HD 128)
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int STAGES = NW * D;                       // warp w owns stages w * D .. w * D + D - 1
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;     // 96 KB in flight per CTA, 2 CTAs per SM
  static_assert(TILE >= 16 && TILE % 16 == 0, "a tile holds a multiple of 16 keys");
  // after the ring: per-warp partial results [NW][G][HD], their (max, sum) [NW][16] each, then the
  // CTA's merged partial [G][HD] and its (max, sum) [16] each, all float
  static constexpr int merge_floats(int G) { return NW * G * HD + 2 * NW * 16 + G * HD + 32; }
  static constexpr int smem_bytes(int G) { return 1024 + RING_BYTES + merge_floats(G) * 4; }
};

// MAXC: the most ranges (CTAs of a cluster) this instantiation merges, 8 or 16: the merge holds that many
// addresses and maxima a thread
template <int HD, int MAXC>
// (head size 64: 168 registers a thread; six warps twice per SM leave 170)
__global__ void __launch_bounds__(DCfg<HD>::THREADS)
attn_decode_kernel(const DecParams p) {
  typedef DCfg<HD> C;
  constexpr int NW = C::NW, D = C::D, THREADS = C::THREADS;
  constexpr int TILE = C::TILE;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  constexpr int CPR = HD / 8;                              // 16-byte chunks per key row
  constexpr int CHUNKS = TILE * CPR / 32;                  // chunks per lane per K (or V) tile
  extern __shared__ uint8_t dsmem_raw[];

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
  const int* bt = p.block_table + (size_t)seq * p.bt_stride;
  const int last_held = pos / p.page_size;
  const int pos_page = bt[last_held];
  const uint32_t ring = smem_u32(smem) + (uint32_t)(warp * D) * C::STAGE_BYTES;   // this warp's stages
  const int lane_r = lane / CPR, lane_ch = lane % CPR;      // this lane's first key row of a tile and its 16 bytes of a row
  const size_t page_stride = (size_t)p.nkv * p.page_size * HD;
  const size_t lane_off = (size_t)kvh * p.page_size * HD + lane_ch * 8;
  bool waited = false;

  // Starts the copies of this warp's tile `i` (the (i / NW)-th of the warp) and closes a copy
  // group, also when there is no such tile, so that the groups can be counted.
  auto issue = [&](int i) {
    if (i < n_tiles) {
      if (tb + i == last_tile && !waited) { pdl_wait(); waited = true; }
      const uint32_t st = ring + (uint32_t)((i / NW) % D) * C::STAGE_BYTES;
      const int j0 = (tb + i) * TILE;
      // A lane copies the same 16 bytes of every (32 / CPR)-th key row. What its addresses share is
      // worked out once per kernel (lane_off, page_stride), and a key's page and place in it are a shift
      // and a mask where the page size is a power of two: the addresses of a tile's 16 copies were some 400
      // instructions a lane, as long as the copies took to arrive.
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int r = lane_r + (32 / CPR) * c;
        const int j = j0 + r;
        // (measured: at head size 128 the divisions are the faster code, 27.3 against 28.4 us for 8 sequences
        // of 4,096 keys; at 64 the shifts, 80.5 against 85.2 us for 64 sequences)
        const bool shifts = HD == 64 && p.page_shift >= 0;
        const int pg_idx = shifts ? (j >> p.page_shift) : j / p.page_size;
        const int off = shifts ? (j & (p.page_size - 1)) : j % p.page_size;
        int page = pg_idx <= last_held ? __ldg(bt + pg_idx) : -1;
        if (page < 0) page = pos_page;
        const size_t src = (size_t)page * page_stride + lane_off + (size_t)(off * HD);
        const uint32_t dst = st + tile_off<TILE>(r, lane_ch);
        cp_async16(dst, p.kcache + src);
        cp_async16(dst + C::KV_BYTES, p.vcache + src);
      }
    }
    cp_async_commit();
  };

  {
    // ------------------------------------------------------------ every warp: fetch, then work
    const int quad = lane >> 2, qi = lane & 3;
    const bool vA = quad < G, vB = quad + 8 < G;
#pragma unroll
    for (int d = 0; d < D; ++d) issue(warp + d * NW);
    if (!waited) { pdl_wait(); waited = true; }   // q comes from the kernel before this one
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

    for (int i = warp; i < n_tiles; i += NW) {
      cp_async_wait<D - 1>();                       // this warp's oldest group, tile i, has landed
      __syncwarp();
      const uint32_t kt = ring + (uint32_t)((i / NW) % D) * C::STAGE_BYTES;
      const uint32_t vt = kt + C::KV_BYTES;
      const int j0 = (tb + i) * TILE;

      // ---- scores: every fragment of the K tile is fetched before the first product, so the
      // shared-memory latencies overlap; rows beyond G hold zeros and are never stored
      uint32_t kf[KSTEPS][TILE / 16][4];
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk)
#pragma unroll
        for (int np = 0; np < TILE / 16; ++np)
          ldsm_x4(kf[kk][np], kt + tile_off<TILE>((2 * np + (mat >> 1)) * 8 + rr, 2 * kk + (mat & 1)));
      float sc[TILE / 8][4];
#pragma unroll
      for (int x = 0; x < TILE / 8; ++x) { sc[x][0] = sc[x][1] = sc[x][2] = sc[x][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int np = 0; np < TILE / 16; ++np) {
          mma16816(sc[2 * np], qf[kk], kf[kk][np][0], kf[kk][np][1]);
          mma16816(sc[2 * np + 1], qf[kk], kf[kk][np][2], kf[kk][np][3]);
        }
      }
      // ---- the V fragments are asked for now and used after the softmax arithmetic
      uint32_t vf[TILE / 16][DTILES / 2][4];
#pragma unroll
      for (int kb = 0; kb < TILE / 16; ++kb)
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp)
          ldsm_x4_t(vf[kb][dp], vt + tile_off<TILE>(kb * 16 + (mat & 1) * 8 + rr, 2 * dp + (mat >> 1)));
      __syncwarp();                                    // everything is in registers: the stage may be refilled
      issue(i + D * NW);
      if (j0 < lo || j0 + TILE - 1 > pos) {        // only a tile at an edge has keys to hide
#pragma unroll
        for (int nt = 0; nt < TILE / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = j0 + nt * 8 + qi * 2 + e;
            if (j > pos || j < lo) { sc[nt][e] = -INFINITY; sc[nt][2 + e] = -INFINITY; }
          }
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < TILE / 8; ++nt) {
        mxA = fmaxf(mxA, fmaxf(sc[nt][0], sc[nt][1]));
        mxB = fmaxf(mxB, fmaxf(sc[nt][2], sc[nt][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      // running maximum in the exp2 domain (the scale is positive, so it commutes with max)
      const float mnA = fmaxf(mA, mxA * p.scale_log2e), mnB = fmaxf(mB, mxB * p.scale_log2e);
      const float useA = (mnA == -INFINITY) ? 0.f : mnA, useB = (mnB == -INFINITY) ? 0.f : mnB;
      if (__any_sync(0xffffffffu, mnA != mA || mnB != mB)) {      // a new maximum somewhere: rescale
        const float corrA = fast_exp2(mA - useA), corrB = fast_exp2(mB - useB);     // exp2(-inf) = 0
        lA *= corrA; lB *= corrB;
#pragma unroll
        for (int x = 0; x < DTILES; ++x) { o[x][0] *= corrA; o[x][1] *= corrA; o[x][2] *= corrB; o[x][3] *= corrB; }
        mA = mnA; mB = mnB;
      }
#pragma unroll
      for (int kb = 0; kb < TILE / 16; ++kb) {
        uint32_t a[4];
        {
          const float sl = p.scale_log2e;
          const float p0 = fast_exp2(fmaf(sc[2 * kb][0], sl, -useA)), p1 = fast_exp2(fmaf(sc[2 * kb][1], sl, -useA));
          const float p2 = fast_exp2(fmaf(sc[2 * kb][2], sl, -useB)), p3 = fast_exp2(fmaf(sc[2 * kb][3], sl, -useB));
          const float p4 = fast_exp2(fmaf(sc[2 * kb + 1][0], sl, -useA)), p5 = fast_exp2(fmaf(sc[2 * kb + 1][1], sl, -useA));
          const float p6 = fast_exp2(fmaf(sc[2 * kb + 1][2], sl, -useB)), p7 = fast_exp2(fmaf(sc[2 * kb + 1][3], sl, -useB));
          lA += p0 + p1 + p4 + p5;
          lB += p2 + p3 + p6 + p7;
          a[0] = pack2(p0, p1); a[1] = pack2(p2, p3);
          a[2] = pack2(p4, p5); a[3] = pack2(p6, p7);
        }
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          mma16816(o[2 * dp], a, vf[kb][dp][0], vf[kb][dp][1]);
          mma16816(o[2 * dp + 1], a, vf[kb][dp][2], vf[kb][dp][3]);
        }
      }
        }
    cp_async_wait<0>();
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

  // ---------------------------------------------------------------- merge the warps
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
    {
      uint32_t bo[MAXC], bm[MAXC], bl[MAXC];
#pragma unroll
      for (int s = 0; s < MAXC; ++s) {
        const uint32_t rk = s < p.splits ? (uint32_t)s : 0u;
        bo[s] = map_to_rank(smem_u32(c_o), rk);
        bm[s] = map_to_rank(smem_u32(c_m), rk);
        bl[s] = map_to_rank(smem_u32(c_l), rk);
      }
      // row r is finished by rank r % splits
      for (int idx = threadIdx.x; idx < G * HD; idx += THREADS) {
        const int r = idx / HD, d = idx % HD;
        if (r % p.splits != rank) continue;
        float ms[MAXC];
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < MAXC; ++s) {
          ms[s] = s < p.splits ? ld_cluster_f32(bm[s] + (uint32_t)r * 4) : -INFINITY;
          M = fmaxf(M, ms[s]);
        }
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s = 0; s < MAXC; ++s) {
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
template <int HD, int MAXC>
int launch_dec_c(const DecParams& p, int num_seqs, cudaStream_t s) {
  typedef DCfg<HD> C;
  static bool configured[64] = {};
  if (allow_dynamic_smem(attn_decode_kernel<HD, MAXC>, C::smem_bytes(16), configured)) return -5;
  if (MAXC > 8) {
    // more than 8 CTAs in a cluster need the kernel's own permission, per device
    static bool wide[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return -5; }
    if (!wide[dev]) {
      if (cudaFuncSetAttribute(attn_decode_kernel<HD, MAXC>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return ERR_BAD_SIZE;
      }
      wide[dev] = true;
    }
  }
  dim3 grid(p.nkv, num_seqs, p.splits);
  if (grid.y > 65535) return ERR_TOO_LARGE;
  return launch_ex(attn_decode_kernel<HD, MAXC>, grid, dim3(C::THREADS), C::smem_bytes(p.nh / p.nkv), s, p.splits, p);
}

template <int HD>
int launch_dec(const DecParams& p, int num_seqs, cudaStream_t s) {
  return p.splits <= 8 ? launch_dec_c<HD, 8>(p, num_seqs, s) : launch_dec_c<HD, 16>(p, num_seqs, s);
}

}  // namespace

// q: [S, ...] bf16, one row per sequence, stride q_stride, head h at h*hd; out likewise.
// kcache / vcache: [num_pages][nkv][page_size][hd] bf16. kv_lens [S]: keys visible to each
// sequence's token (its own included). splits: ranges of keys per sequence (1..16, one cluster).
// `err` is not used (this kernel has no wait that can run out); it keeps the launchers alike.
RLLM_API int rllm_attention_decode(const void* q, int q_stride, const void* kcache, const void* vcache,
                                   long long num_pages, void* out, int out_stride, const int* kv_lens,
                                   const int* block_table, int bt_stride, int num_seqs, int nh, int nkv, int hd,
                                   int page_size, float scale, int window, int splits, int* err, void* stream) {
  (void)err;
  if (num_seqs <= 0) return 0;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || nh / nkv > 16) return ERR_BAD_SIZE;
  if (page_size <= 0 || splits < 1 || splits > MAX_CLUSTER || num_pages <= 0) return ERR_BAD_SIZE;
  if (q_stride % 2 || out_stride % 2 || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) ||
      ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return ERR_BAD_ALIGN;
  DecParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.kv_lens = kv_lens; p.block_table = block_table; p.bt_stride = bt_stride; p.nh = nh; p.nkv = nkv;
  p.page_size = page_size; p.window = window; p.splits = splits; p.scale_log2e = scale * 1.4426950408889634f;
  p.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft) if ((1 << sft) == page_size) p.page_shift = sft;
  cudaStream_t s = (cudaStream_t)stream;
  return hd == 64 ? launch_dec<64>(p, num_seqs, s) : launch_dec<128>(p, num_seqs, s);
}
