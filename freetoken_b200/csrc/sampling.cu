// Next-token choice from float32 logits: greedy, temperature, top-k, top-p.
//
// The reference takes argmax when the whole batch is greedy and otherwise
// softmax(logits / T) followed by an inverse-CDF draw, filtered by top-k then
// top-p when a request sets them (python/freetoken/engine/sample.py:24-80).
// Here every row carries its own temperature, top-k, top-p and uniform number,
// so a row's token does not depend on what else is in the batch:
//   T <= 0            -> argmax, lowest index on ties
//   p_i  = exp((x_i - max) / T)
//   top-k: keep the k largest p (ties at the k-th value are all kept)
//   top-p: of those, keep the smallest set of largest p whose mass reaches
//          top_p of the kept mass (ties at the cut are all kept)
//   draw:  first index whose running kept mass exceeds u * kept mass
#include "common.cuh"

namespace ft {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ float block_max_f(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = scratch[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, scratch[w]);
    scratch[32] = m;
  }
  __syncthreads();
  return scratch[32];
}

// Sum of p_i >= threshold, and how many there are.
__device__ __forceinline__ void kept_mass(const float* p, int V, float thr, float* scratch,
                                          float* mass, float* count) {
  float s = 0.f, c = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = p[i];
    if (v >= thr) { s += v; c += 1.f; }
  }
  *mass = block_sum(s, scratch);
  *count = block_sum(c, scratch);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out, float* __restrict__ probs,
              int V) {
  __shared__ float scratch[33];
  __shared__ float prefix[SAMPLE_THREADS];
  __shared__ int winner;
  pdl_wait();

  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * V;
  const float T = temperature ? temperature[row] : 0.f;

  // one pass: a thread walks its indices in ascending order, so a strictly larger value
  // keeps the first index that holds the thread's maximum
  float mx = -INFINITY;
  int best = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (v > mx) { mx = v; best = i; }
  }
  const float mine = mx;
  mx = block_max_f(mx, scratch);

  if (!(T > 0.f)) {
    if (threadIdx.x == 0) winner = 0x7fffffff;
    __syncthreads();
    if (mine == mx && best != 0x7fffffff) atomicMin(&winner, best);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = winner == 0x7fffffff ? 0 : winner;
    return;
  }

  float* p = probs + (size_t)row * V;
  const float inv_t = 1.f / T;
  for (int i = threadIdx.x; i < V; i += blockDim.x) p[i] = expf((x[i] - mx) * inv_t);
  __syncthreads();

  float thr = 0.f, mass, count;
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V) {
    // Largest threshold that still keeps at least k entries; p lies in [0,1],
    // where float order equals the order of the bit patterns.
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      kept_mass(p, V, __uint_as_float(mid), scratch, &mass, &count);
      if (count >= (float)k) lo = mid; else hi = mid - 1u;
    }
    thr = __uint_as_float(lo);
  }
  const float pp = top_p ? top_p[row] : 1.f;
  if (pp < 1.f) {
    kept_mass(p, V, thr, scratch, &mass, &count);
    const float want = pp * mass;
    unsigned lo = __float_as_uint(thr), hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      kept_mass(p, V, __uint_as_float(mid), scratch, &mass, &count);
      if (mass >= want) lo = mid; else hi = mid - 1u;
    }
    thr = __uint_as_float(lo);
  }

  // Inverse CDF over the kept entries in index order: thread i owns a
  // contiguous chunk, chunk sums are scanned serially, one thread finishes.
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * chunk), end = min(V, begin + chunk);
  float local = 0.f;
  for (int i = begin; i < end; ++i) if (p[i] >= thr) local += p[i];
  prefix[threadIdx.x] = local;
  if (threadIdx.x == 0) winner = 0x7fffffff;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      const float v = prefix[i];
      prefix[i] = run;
      run += v;
    }
    scratch[32] = run;
  }
  __syncthreads();
  const float total = scratch[32];
  const float target = uniform[row] * total;
  const float before = prefix[threadIdx.x];
  if (local > 0.f && before <= target && target < before + local) {
    float run = before;
    int pick = -1, last = -1;
    for (int i = begin; i < end; ++i) {
      if (p[i] >= thr) {
        run += p[i];
        last = i;
        if (run > target) { pick = i; break; }
      }
    }
    atomicMin(&winner, pick >= 0 ? pick : last);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (winner == 0x7fffffff) {
      // u * total rounded up to the total: take the last kept entry
      int last = 0;
      for (int i = V - 1; i >= 0; --i) if (p[i] >= thr) { last = i; break; }
      winner = last;
    }
    out[row] = winner;
  }
}

}  // namespace ft

using namespace ft;

// probs: scratch of [rows, V] floats (unused for greedy rows).
extern "C" int ft_sample(const float* logits, const float* temperature, const int* top_k,
                         const float* top_p, const float* uniform, int* out, float* probs,
                         int rows, int V, cudaStream_t stream) {
  if (rows <= 0) return FT_OK;
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, temperature, top_k, top_p, uniform,
                                                      out, probs, V);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// ------------------------------------------------- no-allocation entry point
// See sampling_static.h.  The scratch lives in the library image; host code
// only ever sees the symbol as a handle, so the device address is looked up
// once per device (with that device current) and handed to the kernel.
#include <mutex>

#include "sampling_static.h"

static __device__ __align__(256) float ft_sample_static_scratch[FT_SAMPLE_STATIC_FLOATS];

static float* ft_sample_static_address(int* error) {
  static float* address[64] = {nullptr};
  static std::mutex guard;            // two host threads may make their first call at once
  std::lock_guard<std::mutex> hold(guard);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) { *error = (int)e; return nullptr; }
  if (device < 0 || device >= 64) { *error = FT_ERR_SHAPE; return nullptr; }
  if (!address[device]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, ft_sample_static_scratch);
    if (e != cudaSuccess) { *error = (int)e; return nullptr; }
    address[device] = static_cast<float*>(p);
  }
  *error = FT_OK;
  return address[device];
}

extern "C" int ft_sample_static(const float* logits, const float* temperature, const int* top_k,
                                const float* top_p, const float* uniform, int* out, int rows,
                                int vocab, cudaStream_t stream) {
  if (rows <= 0) return FT_OK;
  if (vocab <= 0) return FT_ERR_SHAPE;
  if ((long long)rows * (long long)vocab > (long long)FT_SAMPLE_STATIC_FLOATS)
    return FT_ERR_STATIC_TOO_LARGE;
  if (temperature && !uniform) return FT_ERR_SHAPE;
  int error = FT_OK;
  float* scratch = ft_sample_static_address(&error);
  if (!scratch) return error;
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, temperature, top_k, top_p, uniform,
                                                      out, scratch, vocab);
  FT_LAUNCH_CHECK();
  return FT_OK;
}
