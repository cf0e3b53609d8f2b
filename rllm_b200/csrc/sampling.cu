// Token selection from float logits [R, V]: greedy argmax (lowest index wins a
// tie) and the reference's sampling pipeline
//   x/T -> top-k mask -> softmax -> min-p -> top-p -> inverse CDF in vocabulary order
// (src/model/sampler.rs:361-499).
//
// Argmax: the row is cut over a cluster of CTAs, rank 0 picks among the ranks' candidates through
// distributed shared memory. Sampling: the row lies in the shared memory of a cluster of up to
// 8 CTAs (one read of the logits). Instead of sorting, top-k and top-p find their thresholds on
// the order-preserving bit pattern of a float ("the k-th largest logit", "the largest probability
// tau such that the mass of {p >= tau} reaches top_p"), eight candidate thresholds a pass; prefix
// sums over the cluster replace serial walks. Ties at a threshold are all kept, as in
// sampler.rs:397-403. Rows too long for a cluster's shared memory run the one-block-per-row
// kernels, which recompute the probabilities from the logits in every pass.
#include "common.cuh"
#include "sm100.cuh"
#include <type_traits>
using namespace rllm;

namespace {

constexpr int THREADS = 1024;

// monotone map float -> uint32 (order-preserving)
__device__ __forceinline__ unsigned f2key(float f) {
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(unsigned k) {
  unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// One row of the logits is shared by the CTAs of a thread-block cluster along z (ARGMAX_SPLIT
// of them for a large vocabulary, one otherwise); each takes a contiguous range, and rank 0
// picks among the ranks' candidates through distributed shared memory. The rule "largest value,
// lowest index among equals, NaN never wins" holds at every level, so the result does not
// depend on how the row is cut.
constexpr int ARGMAX_SPLIT = 8;

__device__ __forceinline__ void argmax_take(float& best, int& bi, float v, int i) {
  if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, int splits) {
  pdl_launch();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cand_v;
  __shared__ int cand_i;
  const int rank = splits > 1 ? (int)sm100::cluster_rank() : 0;
  const float* x = logits + (size_t)blockIdx.x * V;
  // ranges start on multiples of 4 so that the vector loads stay aligned
  const int per = ((V + splits - 1) / splits + 3) & ~3;
  const int b = min(V, rank * per), e = min(V, b + per);
  float best = -INFINITY; int bi = 0x7fffffff;
  if ((V & 3) == 0 && ((uintptr_t)logits & 15) == 0) {
    const int e4 = b + ((e - b) & ~3);
    for (int i = b + threadIdx.x * 4; i < e4; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      argmax_take(best, bi, v.x, i); argmax_take(best, bi, v.y, i + 1);
      argmax_take(best, bi, v.z, i + 2); argmax_take(best, bi, v.w, i + 3);
    }
    for (int i = e4 + threadIdx.x; i < e; i += blockDim.x) argmax_take(best, bi, x[i], i);
  } else {
    for (int i = b + threadIdx.x; i < e; i += blockDim.x) argmax_take(best, bi, x[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_take(best, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_take(best, bi, ov, oi);
    }
    if (lane == 0) { cand_v = best; cand_i = bi; }
  }
  if (splits > 1) {
    sm100::cluster_sync_all();                 // every rank's candidate is in its shared memory
    if (rank == 0 && threadIdx.x == 0) {
      best = cand_v; bi = cand_i;
      for (int r = 1; r < splits; ++r) {
        const float ov = sm100::ld_cluster_f32(sm100::map_to_rank(sm100::smem_u32(&cand_v), (uint32_t)r));
        const int oi = (int)sm100::ld_cluster_u32(sm100::map_to_rank(sm100::smem_u32(&cand_i), (uint32_t)r));
        argmax_take(best, bi, ov, oi);
      }
      out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
    sm100::cluster_sync_all();                 // nobody leaves while rank 0 still reads
  } else if (threadIdx.x == 0) {
    out[blockIdx.x] = (cand_i == 0x7fffffff) ? 0 : cand_i;
  }
}

__device__ __forceinline__ float block_sum_f(float v, float* red) { return block_sum(v, red); }

__device__ __forceinline__ int block_sum_i(int v, int* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float redf[32];
  __shared__ int redi[32];
  __shared__ float seg[THREADS];
  __shared__ int pick_thread;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * V;
  const float T = temperature[row];
  if (!(T > 0.f)) return;            // a greedy row: the caller has put its argmax into out[row] already
  const float invT = 1.f / T;
  const int tid = threadIdx.x;

  // 1. top-k threshold on the scaled logits (k-th largest; ties kept)
  float thr = -INFINITY;
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V) {
    unsigned lo = 0u, hi = 0xffffffffu;      // largest key with count(key' >= key) >= k
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + 1u;
      int c = 0;
      for (int i = tid; i < V; i += THREADS) c += (f2key(x[i] * invT) >= mid);
      c = block_sum_i(c, redi);
      if (c >= k) lo = mid; else hi = mid - 1u;
    }
    thr = key2f(lo);
  }
  // 2. softmax over the kept logits
  float mx = -INFINITY;
  for (int i = tid; i < V; i += THREADS) { const float v = x[i] * invT; if (v >= thr) mx = fmaxf(mx, v); }
  mx = block_max(mx, redf);
  float sum = 0.f;
  for (int i = tid; i < V; i += THREADS) { const float v = x[i] * invT; if (v >= thr) sum += expf(v - mx); }
  sum = block_sum_f(sum, redf);
  // 3. min-p: drop p < min_p * max p. With e = exp(v - max) the largest e is 1, so the
  //    rule is e < min_p, exact in the e domain; renormalise over what is kept.
  const float emin = min_p ? fmaxf(min_p[row], 0.f) : 0.f;
#define EXPV(i) ((x[i] * invT >= thr) ? expf(x[i] * invT - mx) : 0.f)
  if (emin > 0.f) {
    float kept = 0.f;
    for (int i = tid; i < V; i += THREADS) { const float e = EXPV(i); if (e >= emin) kept += e; }
    sum = block_sum_f(kept, redf);
  }
  const float inv_sum = 1.f / sum;
#define PROB(i) ([&]() { const float e_ = EXPV(i); return e_ >= emin ? e_ * inv_sum : 0.f; }())
  // 4. top-p: largest tau with mass{p >= tau} >= top_p
  const float tp = top_p ? top_p[row] : 1.f;
  float tau = 0.f;
  float mass = 1.f;
  if (tp < 1.f) {
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + 1u;
      const float cand = __uint_as_float(mid);
      float ms = 0.f;
      for (int i = tid; i < V; i += THREADS) { const float p = PROB(i); if (p >= cand) ms += p; }
      ms = block_sum_f(ms, redf);
      if (ms >= tp) lo = mid; else hi = mid - 1u;
    }
    tau = __uint_as_float(lo);
    float ms = 0.f;
    for (int i = tid; i < V; i += THREADS) { const float p = PROB(i); if (p >= tau) ms += p; }
    mass = block_sum_f(ms, redf);
  }
  // 5. inverse CDF in vocabulary order: first i with cumulative > u * mass
  const int per = (V + THREADS - 1) / THREADS;
  const int b = tid * per, e = min(V, b + per);
  float local = 0.f;
  for (int i = b; i < e; ++i) { const float p = PROB(i); if (p >= tau && p > 0.f) local += p; }
  seg[tid] = local;
  if (tid == 0) pick_thread = -1;
  __syncthreads();
  if (tid == 0) {
    const float target = uniform[row] * mass;
    float cum = 0.f; int last = -1;
    for (int i = 0; i < THREADS; ++i) {
      if (seg[i] > 0.f) last = i;
      if (cum + seg[i] > target) { pick_thread = i; redf[0] = cum; break; }
      cum += seg[i];
    }
    redf[1] = target;
    // rounding left none above the target: the last entry with mass is taken
    if (pick_thread < 0) { pick_thread = last < 0 ? 0 : last; redf[0] = 0.f; redf[1] = INFINITY; }
  }
  __syncthreads();
  if (tid == pick_thread) {
    float cum = redf[0]; const float target = redf[1];
    int chosen = -1, last = -1;
    for (int i = b; i < e; ++i) {
      const float p = PROB(i);
      if (!(p >= tau && p > 0.f)) continue;
      last = i;
      cum += p;
      if (cum > target) { chosen = i; break; }
    }
    out[row] = chosen >= 0 ? chosen : (last >= 0 ? last : 0);
  }
#undef PROB
#undef EXPV
}


// ---------------------------------------------------------------------------------------------
// The same pipeline with the row kept in shared memory: the CTAs of a cluster (up to 8 along z)
// take a slice of the vocabulary each, hold its scaled logits (then its probabilities) in shared
// memory, and every reduction runs block -> cluster through distributed shared memory, the ranks'
// parts always added in rank order, so that every CTA gets the same bits and takes the same way.
// The two thresholds (k-th largest logit; the largest probability tau with mass{p >= tau} >= top_p)
// are found on the bit pattern of a float as in the kernel above, but with eight probes a pass,
// which narrows the interval ninefold: 11 passes instead of 32, over shared memory instead of L2.
constexpr int SAMPLE_SPLIT = 8;            // CTAs per row at most
constexpr int SAMPLE_SLICE_MAX = 32768;    // floats of the row a CTA keeps (128 KB)
constexpr int WAYS = 8;                    // probes per pass

struct SampleShared {
  float red_f[32][WAYS];
  int red_i[32][WAYS];
  float part_f[2][WAYS];     // this CTA's parts of a reduction, by parity of the reduction's number
  int part_i[2][WAYS];
  float tot_f[WAYS];
  int tot_i[WAYS];
  int pick_thread, last_thread;
};

// v[j] of every thread of every CTA of the cluster added up (MAX: the largest), same result everywhere.
// `seq` counts the reductions of the kernel: the parts are double-buffered by its parity, so that one
// cluster barrier a reduction is enough (a rank two reductions ahead cannot exist: it needs this one's result).
template <typename T, bool MAX>
__device__ __forceinline__ void cluster_reduce(T (&v)[WAYS], T (*red)[WAYS], T (*part)[WAYS], T* tot, int& seq,
                                               int splits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto join = [](T a, T b) { return MAX ? (b > a ? b : a) : a + b; };
#pragma unroll
  for (int j = 0; j < WAYS; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[j] = join(v[j], __shfl_xor_sync(0xffffffffu, v[j], o));
  }
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < WAYS; ++j) red[warp][j] = v[j];
  }
  __syncthreads();
  const int par = seq & 1;
  if (warp < WAYS) {                               // warp j joins the 32 warps' values of probe j
    T a = red[lane][warp];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = join(a, __shfl_xor_sync(0xffffffffu, a, o));
    if (lane == 0) part[par][warp] = a;
  }
  if (splits > 1) {
    sm100::cluster_sync_all();                     // every rank's parts are written (and visible)
    if (warp == 0) {
      // lane = 8 (r & 3) + j reads the parts of ranks r and r + 4 for probe j; two exchanges join the four pairs
      const int j = lane & 7, r = lane >> 3;
      auto remote = [&](int rr) -> T {
        if (rr >= splits) return MAX ? (T)-INFINITY : (T)0;
        const uint32_t addr = sm100::map_to_rank(sm100::smem_u32(&part[par][j]), (uint32_t)rr);
        if constexpr (std::is_same<T, float>::value) return sm100::ld_cluster_f32(addr);
        else return (T)sm100::ld_cluster_u32(addr);
      };
      T a = join(remote(r), remote(r + 4));
      a = join(a, __shfl_xor_sync(0xffffffffu, a, 8));
      a = join(a, __shfl_xor_sync(0xffffffffu, a, 16));
      if (lane < WAYS) tot[lane] = a;
    }
  } else {
    __syncthreads();
    if (threadIdx.x < WAYS) tot[threadIdx.x] = part[par][threadIdx.x];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < WAYS; ++j) v[j] = tot[j];
  ++seq;
  __syncthreads();                                  // tot and red may be written again
}

// probes t_1 < ... < t_WAYS in (lo, hi], evenly spread (clipped to hi when the interval is short)
__device__ __forceinline__ void probes(unsigned lo, unsigned hi, unsigned (&t)[WAYS]) {
  const unsigned long long span = (unsigned long long)hi - lo;          // >= 1
  const unsigned long long step = span / (WAYS + 1) > 0 ? span / (WAYS + 1) : 1;
#pragma unroll
  for (int j = 0; j < WAYS; ++j) {
    const unsigned long long x = (unsigned long long)lo + (unsigned long long)(j + 1) * step;
    t[j] = x > hi ? hi : (unsigned)x;
  }
}

__global__ void __launch_bounds__(THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                      const float* __restrict__ min_p, const float* __restrict__ uniform,
                      int* __restrict__ out, int splits, int per) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float vals[];                  // the slice: scaled logits, later probabilities
  __shared__ SampleShared sh;
  const int row = blockIdx.x;
  const float T = temperature[row];
  if (!(T > 0.f)) return;            // a greedy row (the same for every CTA of its cluster): out[row] holds its argmax
  const float invT = 1.f / T;
  const int tid = threadIdx.x;
  const int rank = splits > 1 ? (int)sm100::cluster_rank() : 0;
  const int b = min(V, rank * per), n = min(V, b + per) - b;
  const float* x = logits + (size_t)row * V + b;
  for (int i = tid; i < n; i += THREADS) vals[i] = x[i] * invT;
  __syncthreads();
  int seq = 0;
  float f8[WAYS];
  int i8[WAYS];

  // 1. top-k threshold on the scaled logits: the largest key t with count{key >= t} >= k (ties kept)
  float thr = -INFINITY;
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V) {
    unsigned lo = 0u, hi = 0xffffffffu;
    while (lo < hi) {
      unsigned t[WAYS];
      probes(lo, hi, t);
#pragma unroll
      for (int j = 0; j < WAYS; ++j) i8[j] = 0;
      for (int i = tid; i < n; i += THREADS) {
        const unsigned key = f2key(vals[i]);
#pragma unroll
        for (int j = 0; j < WAYS; ++j) i8[j] += (key >= t[j]);
      }
      cluster_reduce<int, false>(i8, sh.red_i, sh.part_i, sh.tot_i, seq, splits);
      int best = -1;                                // the largest probe that still has k at or above it
#pragma unroll
      for (int j = 0; j < WAYS; ++j) if (i8[j] >= k) best = j;
      const unsigned nlo = best >= 0 ? t[best] : lo;
      const unsigned nhi = best == WAYS - 1 ? hi : t[best + 1] - 1u;
      lo = nlo; hi = nhi < nlo ? nlo : nhi;
    }
    thr = key2f(lo);
  }
  // 2. softmax over the kept logits: e = exp(v - max), 0 for the dropped
#pragma unroll
  for (int j = 0; j < WAYS; ++j) f8[j] = -INFINITY;
  for (int i = tid; i < n; i += THREADS) { const float v = vals[i]; if (v >= thr) f8[0] = fmaxf(f8[0], v); }
  cluster_reduce<float, true>(f8, sh.red_f, sh.part_f, sh.tot_f, seq, splits);
  const float mx = f8[0];
  const float emin = min_p ? fmaxf(min_p[row], 0.f) : 0.f;
#pragma unroll
  for (int j = 0; j < WAYS; ++j) f8[j] = 0.f;
  for (int i = tid; i < n; i += THREADS) {
    const float v = vals[i];
    const float e = v >= thr ? expf(v - mx) : 0.f;
    vals[i] = e;
    f8[0] += e;
    // 3. min-p: drop p < min_p * max p. The largest e is 1, so the rule is e < min_p, exact in the e domain
    if (e >= emin) f8[1] += e;
  }
  cluster_reduce<float, false>(f8, sh.red_f, sh.part_f, sh.tot_f, seq, splits);
  const float inv_sum = 1.f / (emin > 0.f ? f8[1] : f8[0]);
  for (int i = tid; i < n; i += THREADS) { const float e = vals[i]; vals[i] = e >= emin ? e * inv_sum : 0.f; }
  __syncthreads();
  // 4. top-p: the largest tau with mass{p >= tau} >= top_p
  const float tp = top_p ? top_p[row] : 1.f;
  float tau = 0.f, mass = 1.f;
  if (tp < 1.f) {
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      unsigned t[WAYS];
      probes(lo, hi, t);
#pragma unroll
      for (int j = 0; j < WAYS; ++j) f8[j] = 0.f;
      for (int i = tid; i < n; i += THREADS) {
        const float pr = vals[i];
#pragma unroll
        for (int j = 0; j < WAYS; ++j) if (pr >= __uint_as_float(t[j])) f8[j] += pr;
      }
      cluster_reduce<float, false>(f8, sh.red_f, sh.part_f, sh.tot_f, seq, splits);
      int best = -1;
#pragma unroll
      for (int j = 0; j < WAYS; ++j) if (f8[j] >= tp) best = j;
      const unsigned nlo = best >= 0 ? t[best] : lo;
      const unsigned nhi = best == WAYS - 1 ? hi : t[best + 1] - 1u;
      lo = nlo; hi = nhi < nlo ? nlo : nhi;
    }
    tau = __uint_as_float(lo);
  }
  // 5. inverse CDF in vocabulary order: the first i with cumulative > u * mass. Every thread adds up a
  //    run of consecutive entries, every CTA its slice; the slices before this one give its offset.
  const int per_t = (n + THREADS - 1) / THREADS;
  const int tb = min(n, tid * per_t), te = min(n, tb + per_t);
  float local = 0.f;
  for (int i = tb; i < te; ++i) { const float pr = vals[i]; if (pr >= tau && pr > 0.f) local += pr; }
  // the masses before each thread's run, in a fixed order: lanes within a warp, then the warps
  const int lane = tid & 31, warp = tid >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
  if (lane == 31) sh.red_f[warp][0] = incl;
  if (tid == 0) { sh.pick_thread = 0x7fffffff; sh.last_thread = -1; }
  __syncthreads();
  if (warp == 0) {
    const float w = sh.red_f[lane][0];              // THREADS / 32 = 32 warps
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float t = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += t; }
    sh.red_f[lane][1] = wi - w;
    if (lane == 31) sh.part_f[seq & 1][0] = wi;     // the slice's mass
  }
  __syncthreads();
  const float excl = sh.red_f[warp][1] + (incl - local);
  float slice_mass[SAMPLE_SPLIT];
  if (splits > 1) sm100::cluster_sync_all();
  for (int r = 0; r < splits; ++r)
    slice_mass[r] = splits > 1 ? sm100::ld_cluster_f32(sm100::map_to_rank(sm100::smem_u32(&sh.part_f[seq & 1][0]), (uint32_t)r))
                               : sh.part_f[seq & 1][0];
  ++seq;
  mass = 0.f;
  for (int r = 0; r < splits; ++r) mass += slice_mass[r];
  const float target = uniform[row] * mass;
  // which slice holds the target; if rounding leaves none above it, the last slice with mass
  int owner = -1, last_with_mass = -1;
  float before = 0.f, before_owner = 0.f;
  for (int r = 0; r < splits; ++r) {
    if (slice_mass[r] > 0.f) last_with_mass = r;
    if (owner < 0 && before + slice_mass[r] > target) { owner = r; before_owner = before; }
    before += slice_mass[r];
  }
  const bool fallback = owner < 0;
  if (fallback) owner = last_with_mass < 0 ? 0 : last_with_mass;
  if (rank == owner) {
    // the first thread whose run takes the cumulative mass past the target; else the last one with mass
    const float cum0 = before_owner + excl;
    if (local > 0.f) {
      atomicMax(&sh.last_thread, tid);
      if (!fallback && cum0 + local > target) atomicMin(&sh.pick_thread, tid);
    }
    __syncthreads();
    const bool none = sh.pick_thread == 0x7fffffff;
    const int pick = none ? (sh.last_thread < 0 ? 0 : sh.last_thread) : sh.pick_thread;
    if (tid == pick) {
      float cum = none ? 0.f : cum0;
      const float tgt = none ? INFINITY : target;
      int chosen = -1, last = -1;
      for (int i = tb; i < te; ++i) {
        const float pr = vals[i];
        if (!(pr >= tau && pr > 0.f)) continue;
        last = i;
        cum += pr;
        if (cum > tgt) { chosen = i; break; }
      }
      out[row] = b + (chosen >= 0 ? chosen : (last >= 0 ? last : 0));
    }
  }
  if (splits > 1) sm100::cluster_sync_all();        // nobody leaves while another rank may still read its parts
}

}  // namespace

// logits[rows[i], cols[i]] += vals[i], i < n (the penalties of tokens already produced: a handful of
// entries; the three lists may lie in pinned host memory). (row, col) pairs are distinct.
__global__ void add_at_kernel(float* __restrict__ logits, int V, const int* __restrict__ rows,
                              const int* __restrict__ cols, const float* __restrict__ vals, int n) {
  pdl_launch();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    logits[(size_t)rows[i] * V + cols[i]] += vals[i];
}

RLLM_API int rllm_add_at(float* logits, int R, int V, const int* rows, const int* cols, const float* vals, int n,
                         void* stream) {
  if (n <= 0) return 0;
  if (R <= 0 || V <= 0) return ERR_BAD_SIZE;
  const int blocks = (n + 255) / 256 < 64 ? (n + 255) / 256 : 64;
  return launch_ex(add_at_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 1, logits, V, rows, cols, vals, n);
}

// Log-probabilities of the distribution the draw starts from: softmax of x/T (x itself for a greedy
// row) over the logits that top-k keeps, before min-p and top-p (src/model/sampler.rs:421-428,
// 501-541). One block per listed row: lp[i][0] = ln p(chosen[row]) (-inf if top-k dropped it),
// lp[i][1 + j] and ids[i][j] = the j-th most probable token, j < n_top, equals by rising index;
// where fewer than n_top tokens are kept the rest is (-inf, -1).
constexpr int TOP_LOGPROBS_MAX = 20;

// f(value, index) for every entry of a row, four a load where the row allows it (the passes below
// wait for L2, not for arithmetic: independent wide loads are what shortens them)
template <typename F>
__device__ __forceinline__ void row_for_each(const float* __restrict__ x, int V, F f) {
  const int tid = threadIdx.x;
  if ((V & 3) == 0 && ((uintptr_t)x & 15) == 0) {
#pragma unroll 2
    for (int i = tid * 4; i < V; i += THREADS * 4) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      f(v.x, i); f(v.y, i + 1); f(v.z, i + 2); f(v.w, i + 3);
    }
  } else {
    for (int i = tid; i < V; i += THREADS) f(x[i], i);
  }
}

__global__ void __launch_bounds__(THREADS)
logprobs_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                const int* __restrict__ top_k, const int* __restrict__ chosen, const int* __restrict__ rows,
                int n_top, float* __restrict__ lp, int* __restrict__ ids) {
  pdl_launch();
  pdl_wait();
  __shared__ float redf[32];
  __shared__ int redi[32];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float pick_v;
  __shared__ int pick_i;
  const int row = rows[blockIdx.x];
  const float* x = logits + (size_t)row * V;
  const float T = temperature[row];
  const float invT = T > 0.f ? 1.f / T : 1.f;
  const int tid = threadIdx.x;
  float thr = -INFINITY;
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V) {
    unsigned lo = 0u, hi = 0xffffffffu;      // largest key with count(key' >= key) >= k
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + 1u;
      int c = 0;
      row_for_each(x, V, [&](float xv, int) { c += (f2key(xv * invT) >= mid); });
      c = block_sum_i(c, redi);
      if (c >= k) lo = mid; else hi = mid - 1u;
    }
    thr = key2f(lo);
  }
  float mx = -INFINITY;
  row_for_each(x, V, [&](float xv, int) { const float v = xv * invT; if (v >= thr) mx = fmaxf(mx, v); });
  mx = block_max(mx, redf);
  float sum = 0.f;
  row_for_each(x, V, [&](float xv, int) { const float v = xv * invT; if (v >= thr) sum += expf(v - mx); });
  sum = block_sum_f(sum, redf);
  const float lse = mx + logf(sum);
  float* lp_row = lp + (size_t)blockIdx.x * (1 + n_top);
  int* id_row = ids + (size_t)blockIdx.x * (n_top > 0 ? n_top : 1);
  if (tid == 0) {
    const int c = chosen[row];
    const float v = (c >= 0 && c < V) ? x[c] * invT : -INFINITY;
    lp_row[0] = v >= thr ? v - lse : -INFINITY;
  }
  // the n_top largest, one pass each: the largest (value, then lowest index) that comes after the last pick
  float last_v = INFINITY; int last_i = -1;
  for (int j = 0; j < n_top; ++j) {
    float best = -INFINITY; int bi = 0x7fffffff;
    row_for_each(x, V, [&](float xv, int i) {
      const float v = xv * invT;
      if (v >= thr && (v < last_v || (v == last_v && i > last_i))) argmax_take(best, bi, v, i);
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_take(best, bi, ov, oi);
    }
    const int lane = tid & 31, warp = tid >> 5;
    __syncthreads();                           // the last round's pick has been read by everybody
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      best = sv[lane]; bi = si[lane];          // THREADS / 32 = 32 warps
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(best, bi, ov, oi);
      }
      if (lane == 0) {
        pick_v = best; pick_i = bi;
        const bool found = bi != 0x7fffffff;
        lp_row[1 + j] = found ? best - lse : -INFINITY;
        id_row[j] = found ? bi : -1;
      }
    }
    __syncthreads();
    last_v = pick_v; last_i = pick_i;
    if (last_i == 0x7fffffff) {                // nothing is left: the rest of the list is empty
      if (tid == 0) for (int r = j + 1; r < n_top; ++r) { lp_row[1 + r] = -INFINITY; id_row[r] = -1; }
      break;
    }
  }
}

// rows: the n rows of `logits` (and of temperature, top_k, chosen) that want them; lp float [n, 1 + n_top],
// ids int [n, n_top]. temperature, top_k and rows may lie in pinned host memory.
RLLM_API int rllm_logprobs(const float* logits, int R, int V, const float* temperature, const int* top_k,
                           const int* chosen, const int* rows, int n, int n_top, float* lp, int* ids,
                           void* stream) {
  if (n <= 0) return 0;
  if (R <= 0 || V <= 0 || n_top < 0 || n_top > TOP_LOGPROBS_MAX) return ERR_BAD_SIZE;
  return launch_ex(logprobs_kernel, dim3(n), dim3(THREADS), 0, (cudaStream_t)stream, 1, logits, V, temperature, top_k,
                   chosen, rows, n_top, lp, ids);
}

RLLM_API int rllm_argmax(const float* logits, int R, int V, int* out, void* stream) {
  if (R <= 0) return 0;
  if (V <= 0) return ERR_BAD_SIZE;
  const int splits = V >= 16384 ? ARGMAX_SPLIT : 1;
  return launch_ex(argmax_kernel, dim3(R, 1, splits), dim3(THREADS), 0, (cudaStream_t)stream, splits, logits, V,
                   out, splits);
}

// Per-row parameter arrays of length R; top_k / top_p / min_p may be null (off).
// A row whose temperature is not > 0 is left as it is: the caller runs rllm_argmax into `out` first.
RLLM_API int rllm_sample(const float* logits, int R, int V, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p,
                         const float* uniform, int* out, void* stream) {
  if (R <= 0) return 0;
  if (V <= 0) return ERR_BAD_SIZE;
  // the row in the shared memory of 1 to 8 CTAs; a vocabulary beyond that goes the slow way, through L2
  int splits = 1;
  while (splits < SAMPLE_SPLIT && (V + splits - 1) / splits > SAMPLE_SLICE_MAX / 2) splits *= 2;
  const int per = ((V + splits - 1) / splits + 3) & ~3;
  if (per <= SAMPLE_SLICE_MAX) {
    static bool configured[64] = {};
    if (allow_dynamic_smem(sample_cluster_kernel, SAMPLE_SLICE_MAX * 4, configured)) return -5;
    return launch_ex(sample_cluster_kernel, dim3(R, 1, splits), dim3(THREADS), (size_t)per * 4, (cudaStream_t)stream,
                     splits, logits, V, temperature, top_k, top_p, min_p, uniform, out, splits, per);
  }
  return launch_ex(sample_kernel, dim3(R), dim3(THREADS), 0, (cudaStream_t)stream, 1, logits, V, temperature, top_k, top_p,
                   min_p, uniform, out);
}
