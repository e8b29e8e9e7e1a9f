// Router scoring / top-k, and the deterministic sort of routes by expert.
//
// Router (python/freetoken/models/minimax_m3/moe.py:71-81, softmax variant
// python/freetoken/moe/fused.py:27-31), all float32:
//   s = sigmoid(logits) | softmax(logits);  c = s + bias (bias only chooses)
//   ids = top-k of c (ties: lower expert id);  w = s[ids]
//   renormalise: w /= (sum w + 1e-20);  w *= scale
// Sorting: the reference pads and scatters with atomics, so the order inside an
// expert varies from run to run (python/freetoken/kernel/triton/moe_align.py:18-20).
// Here one warp per expert scans the routes in order: rows of an expert keep
// ascending (token, slot) order, run after run.
#include "common.cuh"

namespace ft {

// Scores and top-k of one token by one warp.  `score` and `choice` are E floats
// of shared memory each.  With k <= 32 lane j < k returns the j-th choice in
// (my_id, my_w); otherwise ids and weights go through `ids_out` / `weights_out`.
__device__ __forceinline__ void select_token(const float* __restrict__ x, const float* __restrict__ bias,
                                             float* score, float* choice, int* ids_out, float* weights_out,
                                             int E, int k, int softmax_scoring, int renormalize, float scale,
                                             int terms, int lane, int& my_id, float& my_w) {
  // a row holds `terms` partial logits per expert, E apart (the router weight
  // split into bfloat16 terms); they are summed in order, in float32.  A lane takes
  // experts lane, lane + 32, ...; it fetches eight of them at a time into registers
  // before it touches shared memory, so that its loads from global memory are in flight
  // together (one after the other they were most of this function's time: each waits
  // for L2)
  constexpr int EPL = 8;
  auto load_logits = [&](int base, float (&v)[EPL]) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = base + i * 32 + lane;
      v[i] = e < E ? x[e] : 0.f;
    }
    for (int p = 1; p < terms; ++p) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = base + i * 32 + lane;
        if (e < E) v[i] += x[p * E + e];
      }
    }
  };
  if (softmax_scoring) {
    float mx = -INFINITY;
    for (int base = 0; base < E; base += 32 * EPL) {
      float v[EPL];
      load_logits(base, v);
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = base + i * 32 + lane;
        if (e < E) { score[e] = v[i]; mx = fmaxf(mx, v[i]); }
      }
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(score[e] - mx);
      score[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) score[e] = score[e] / sum;
  } else {
    for (int base = 0; base < E; base += 32 * EPL) {
      float v[EPL];
      load_logits(base, v);
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = base + i * 32 + lane;
        if (e < E) score[e] = 1.f / (1.f + expf(-v[i]));
      }
    }
  }
  for (int base = 0; base < E; base += 32 * EPL) {
    float b[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = base + i * 32 + lane;
      b[i] = (bias && e < E) ? bias[e] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = base + i * 32 + lane;
      if (e < E) choice[e] = score[e] + b[i];
    }
  }
  __syncwarp();
  float wsum = 0.f;
  my_id = 0;            // lane j keeps the j-th choice (k <= 32), else it goes through memory
  my_w = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (c > best) { best = c; arg = e; }  // ascending e: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;  // all values NaN or -inf: stay in range
    const float w = score[arg];
    wsum += w;
    if (lane == (j & 31)) {
      if (k <= 32) { my_id = arg; my_w = w; }
      else { ids_out[j] = arg; weights_out[j] = w; }
    }
    if (lane == 0) choice[arg] = -INFINITY;
    __syncwarp();
  }
  if (k <= 32) {
    if (renormalize) my_w = my_w / (wsum + 1e-20f);
    my_w *= scale;
  } else if (lane == 0) {
    for (int j = 0; j < k; ++j) {
      float w = weights_out[j];
      if (renormalize) w = w / (wsum + 1e-20f);
      weights_out[j] = w * scale;
    }
  }
}

template <int WARPS>
__global__ void router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                     int* __restrict__ ids, float* __restrict__ weights, int T, int E,
                                     int k, int softmax_scoring, int renormalize, float scale, int terms) {
  extern __shared__ float smem[];  // [WARPS][2][E]: scores, choice values
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();

  const int t = blockIdx.x * WARPS + warp;
  if (t >= T) return;
  float* score = smem + (size_t)warp * 2 * E;
  int my_id;
  float my_w;
  select_token(logits + (size_t)t * E * terms, bias, score, score + E, ids + (size_t)t * k,
               weights + (size_t)t * k, E, k, softmax_scoring, renormalize, scale, terms, lane, my_id, my_w);
  if (k <= 32 && lane < k) {
    ids[(size_t)t * k + lane] = my_id;
    weights[(size_t)t * k + lane] = my_w;
  }
}

// A handful of tokens (a small decode batch): selection and the stable sort of
// the few routes in ONE block and one launch.  Warp t selects for token t; then
// a thread per expert counts its routes by walking the (at most 256) route ids
// in shared memory, one warp scans the counts, and a thread per expert places
// its routes in ascending order.  Same results as router_select + moe_sort.
constexpr int SMALL_WARPS = 8;

__global__ void __launch_bounds__(SMALL_WARPS * 32) route_small_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids,
    float* __restrict__ weights, int* __restrict__ counts, int* __restrict__ offsets,
    int* __restrict__ sorted_route, int* __restrict__ sorted_token, int* __restrict__ active, int T, int E,
    int k, int softmax_scoring, int renormalize, float scale, int terms) {
  extern __shared__ float smem[];  // [T][2][E] scores and choices, then ints: ids [T*k], counts [E], before [E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = T * k;
  int* s_ids = reinterpret_cast<int*>(smem + (size_t)T * 2 * E);
  int* s_cnt = s_ids + R;
  int* s_before = s_cnt + E;
  pdl_wait();

  if (warp < T) {
    int my_id;
    float my_w;
    float* score = smem + (size_t)warp * 2 * E;
    select_token(logits + (size_t)warp * E * terms, bias, score, score + E, nullptr, nullptr, E, k,
                 softmax_scoring, renormalize, scale, terms, lane, my_id, my_w);
    if (lane < k) {
      ids[warp * k + lane] = my_id;
      weights[warp * k + lane] = my_w;
      s_ids[warp * k + lane] = my_id;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int r = 0; r < R; ++r) c += s_ids[r] == e;
    s_cnt[e] = c;
    counts[e] = c;
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive scan over the experts: a lane takes a run of consecutive experts
    const int per = (E + 31) / 32, begin = lane * per, end = min(E, begin + per);
    int rows = 0, busy = 0;
    for (int e = begin; e < end; ++e) { rows += s_cnt[e]; busy += s_cnt[e] > 0; }
    int rows_before = rows, busy_before = busy;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, rows_before, o), b = __shfl_up_sync(0xffffffffu, busy_before, o);
      if (lane >= o) { rows_before += a; busy_before += b; }
    }
    const int total_rows = __shfl_sync(0xffffffffu, rows_before, 31);
    const int total_busy = __shfl_sync(0xffffffffu, busy_before, 31);
    rows_before -= rows;
    busy_before -= busy;
    for (int e = begin; e < end; ++e) {
      s_before[e] = rows_before;
      offsets[e] = rows_before;
      if (s_cnt[e] > 0) active[busy_before++] = e;
      rows_before += s_cnt[e];
    }
    if (lane == 0) {
      offsets[E] = total_rows;
      active[E] = total_busy;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_cnt[e] == 0) continue;
    int at = s_before[e];
    for (int r = 0; r < R; ++r) {
      if (s_ids[r] == e) {
        sorted_route[at] = r;
        sorted_token[at] = r / k;
        ++at;
      }
    }
  }
}

// Router logits for few tokens.  logits[t,e] = sum_h x[t,h] * W[e,h] in
// float32.  One warp owns an expert row and 8 tokens; the row is walked in
// pieces of 256 (a lane holds 8 consecutive values) against the 8 tokens'
// matching pieces; a lane sums its share in ascending h, lanes are added by an
// xor-shuffle tree - the same arithmetic for a token whatever else is in the
// launch.  Needs H % 8 == 0 and 16-byte aligned rows.
__device__ __forceinline__ void load8f(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8f(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename AT>
__global__ void __launch_bounds__(128) router_logits_kernel(const AT* __restrict__ x, long long ldx,
                                                            const float* __restrict__ W,
                                                            float* __restrict__ logits, int T, int E,
                                                            int H) {
  // one block per (expert, 8 tokens); its 4 warps take a quarter of the row
  // each (pieces p = warp, warp+4, ... of 256 values) and their partial sums are
  // added in warp order
  constexpr int TT = 8;
  __shared__ float part[4][TT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.x;
  const int t0 = blockIdx.y * TT;
  pdl_wait();
  const float* w = W + (size_t)e * H;
  float acc[TT];
#pragma unroll
  for (int i = 0; i < TT; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int h = warp * 256 + lane * 8; h < H; h += 1024) {
    float wv[8];
    load8f(w + h, wv);
    float xv[TT][8];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      if (t0 + tt < T) load8f(x + (size_t)(t0 + tt) * ldx + h, xv[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      if (t0 + tt < T) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[tt] = fmaf(xv[tt][i], wv[i], acc[tt]);
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const float v = warp_sum(acc[tt]);
    if (lane == 0) part[warp][tt] = v;
  }
  __syncthreads();
  if (threadIdx.x < TT && t0 + threadIdx.x < T) {
    const int tt = threadIdx.x;
    logits[(size_t)(t0 + tt) * E + e] = ((part[0][tt] + part[1][tt]) + part[2][tt]) + part[3][tt];
  }
}

constexpr int SCAN = 8;  // route ids a lane reads ahead while scanning

// counts[e] = number of routes that chose expert e.  One warp per expert.
__global__ void moe_count_kernel(const int* __restrict__ ids, int* __restrict__ counts, int R, int E) {
  const int lane = threadIdx.x & 31;
  pdl_wait();

  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= E) return;
  int c = 0;
  for (int base = 0; base < R; base += 32 * SCAN) {
    int v[SCAN];                      // SCAN independent loads in flight
#pragma unroll
    for (int u = 0; u < SCAN; ++u) {
      const int r = base + 32 * u + lane;
      v[u] = r < R ? ids[r] : -1;
    }
#pragma unroll
    for (int u = 0; u < SCAN; ++u) c += __popc(__ballot_sync(0xffffffffu, v[u] == e));
  }
  if (lane == 0) counts[e] = c;
}

// offsets[e] = sum counts[<e]; sorted_route[offsets[e] + i] = i-th route of
// expert e in ascending route order; sorted_token = sorted_route / k;
// active[j] = j-th expert that has routes (ascending), active[E] = how many.
__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ counts,
                                   int* __restrict__ offsets, int* __restrict__ sorted_route,
                                   int* __restrict__ sorted_token, int* __restrict__ active,
                                   int R, int E, int k) {
  const int lane = threadIdx.x & 31;
  pdl_wait();

  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= E) return;
  int before = 0, busy_before = 0;
  for (int base = 0; base < e; base += 32) {
    const int i = base + lane;
    const int c = i < e ? counts[i] : 0;
    before += c;
    busy_before += c > 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    busy_before += __shfl_xor_sync(0xffffffffu, busy_before, o);
  }
  if (lane == 0) {
    const int mine = counts[e];
    offsets[e] = before;
    if (mine > 0) active[busy_before] = e;
    if (e == E - 1) {
      offsets[E] = before + mine;
      active[E] = busy_before + (mine > 0);
    }
  }
  int at = before;
  for (int base = 0; base < R; base += 32 * SCAN) {
    int v[SCAN];
#pragma unroll
    for (int u = 0; u < SCAN; ++u) {
      const int r = base + 32 * u + lane;
      v[u] = r < R ? ids[r] : -1;
    }
#pragma unroll
    for (int u = 0; u < SCAN; ++u) {
      const bool hit = v[u] == e;
      const unsigned ballot = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = base + 32 * u + lane;
        const int dst = at + __popc(ballot & ((1u << lane) - 1u));
        sorted_route[dst] = r;
        sorted_token[dst] = r / k;
      }
      at += __popc(ballot);
    }
  }
}


// ---- the same sort for many routes (prompt portions): chunks of 256 routes
// Three launches instead of one warp per expert walking every route:
//   1. per chunk, a histogram over the experts        -> chunk_counts[c][e]
//   2. per expert, the running sum over the chunks    -> chunk_counts[c][e] =
//      routes of e before chunk c; counts, offsets and the active list
//   3. per chunk (one warp), routes are ranked 32 at a time: lanes with the
//      same expert find each other with match.any, a lane's rank is the number
//      of lower lanes among them, the expert's cursor then moves on
// The result is the same stable order (ascending route inside an expert).
constexpr int SORT_CHUNK = 256;

__global__ void __launch_bounds__(SORT_CHUNK) moe_chunk_count_kernel(const int* __restrict__ ids,
                                                                    int* __restrict__ chunk_counts, int R,
                                                                    int E) {
  extern __shared__ int hist[];   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int r = blockIdx.x * SORT_CHUNK + threadIdx.x;
  if (r < R) {
    const int e = ids[r];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_counts[(size_t)blockIdx.x * E + e] = hist[e];
}

// One block.  Experts are taken blockDim at a time, in ascending order, with a
// carry for the offsets and for the number of busy experts.
__global__ void __launch_bounds__(1024) moe_chunk_scan_kernel(int* __restrict__ chunk_counts,
                                                              int* __restrict__ counts, int* __restrict__ offsets,
                                                              int* __restrict__ active, int chunks, int E) {
  __shared__ int scan_rows[1024], scan_busy[1024];
  __shared__ int carry_rows, carry_busy;
  if (threadIdx.x == 0) { carry_rows = 0; carry_busy = 0; }
  __syncthreads();
  for (int base = 0; base < E; base += blockDim.x) {
    const int e = base + threadIdx.x;
    int total = 0;
    if (e < E) {
      // eight chunks' counts are fetched together (one after the other, each behind the
      // store before it, the loads were this kernel's whole time), then turned into prefixes
      for (int c0 = 0; c0 < chunks; c0 += 8) {
        int v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = c0 + u < chunks ? chunk_counts[(size_t)(c0 + u) * E + e] : 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (c0 + u < chunks) chunk_counts[(size_t)(c0 + u) * E + e] = total;
          total += v[u];
        }
      }
      counts[e] = total;
    }
    scan_rows[threadIdx.x] = total;
    scan_busy[threadIdx.x] = total > 0;
    __syncthreads();
    for (int o = 1; o < (int)blockDim.x; o <<= 1) {
      const int a = threadIdx.x >= (unsigned)o ? scan_rows[threadIdx.x - o] : 0;
      const int b = threadIdx.x >= (unsigned)o ? scan_busy[threadIdx.x - o] : 0;
      __syncthreads();
      scan_rows[threadIdx.x] += a;
      scan_busy[threadIdx.x] += b;
      __syncthreads();
    }
    if (e < E) {
      const int before = carry_rows + scan_rows[threadIdx.x] - total;
      offsets[e] = before;
      if (total > 0) active[carry_busy + scan_busy[threadIdx.x] - 1] = e;
      if (e == E - 1) {
        offsets[E] = before + total;
        active[E] = carry_busy + scan_busy[threadIdx.x];
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) {
      carry_rows += scan_rows[threadIdx.x];
      carry_busy += scan_busy[threadIdx.x];
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128) moe_chunk_scatter_kernel(const int* __restrict__ ids,
                                                                const int* __restrict__ chunk_counts,
                                                                const int* __restrict__ offsets,
                                                                int* __restrict__ sorted_route,
                                                                int* __restrict__ sorted_token, int R, int E,
                                                                int k, int chunks) {
  extern __shared__ int cursors[];   // [warps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * (blockDim.x >> 5) + warp;
  if (c >= chunks) return;
  int* cursor = cursors + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) cursor[e] = offsets[e] + chunk_counts[(size_t)c * E + e];
  __syncwarp();
  const int first = c * SORT_CHUNK;
  for (int it = 0; it < SORT_CHUNK / 32; ++it) {
    const int r = first + it * 32 + lane;
    int e = r < R ? ids[r] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int at = 0;
    if (e >= 0) at = cursor[e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) cursor[e] += __popc(peers);
    __syncwarp();
    if (e >= 0) {
      sorted_route[at] = r;
      sorted_token[at] = r / k;
    }
  }
}

}  // namespace ft

using namespace ft;

extern "C" {

int ft_router_select(const float* logits, const float* bias, int* ids, float* weights, int T,
                     int E, int k, int softmax_scoring, int renormalize, float scale, int terms,
                     cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (k <= 0 || k > E || terms < 1) return FT_ERR_SHAPE;
  constexpr int WARPS = 4;
  const size_t smem = (size_t)WARPS * 2 * E * sizeof(float);
  if (smem > 200 * 1024) return FT_ERR_SHAPE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(router_select_kernel<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(router_select_kernel<WARPS>, dim3((T + WARPS - 1) / WARPS), dim3(WARPS * 32), smem, stream,
             logits, bias, ids, weights, T, E, k, softmax_scoring, renormalize, scale, terms);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// router_select + moe_sort in one launch; T <= 8 tokens, k <= 32.
int ft_route_small(const float* logits, const float* bias, int* ids, float* weights, int* counts,
                   int* offsets, int* sorted_route, int* sorted_token, int* active, int T, int E, int k,
                   int softmax_scoring, int renormalize, float scale, int terms, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (T > SMALL_WARPS || k <= 0 || k > 32 || k > E || terms < 1) return FT_ERR_SHAPE;
  const size_t smem = (size_t)T * 2 * E * sizeof(float) + ((size_t)T * k + 2 * (size_t)E) * sizeof(int);
  if (smem > 160 * 1024) return FT_ERR_SHAPE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(route_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(route_small_kernel, dim3(1), dim3(SMALL_WARPS * 32), smem, stream, logits, bias, ids, weights,
             counts, offsets, sorted_route, sorted_token, active, T, E, k, softmax_scoring, renormalize, scale,
             terms);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_router_logits(const void* x, int x_dtype, long long ldx, const float* W, float* logits,
                     int T, int E, int H, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if ((H & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return FT_ERR_SHAPE;
  dim3 grid(E, (T + 7) / 8);
  FT_DISPATCH(x_dtype, AT,
              launch_pdl(router_logits_kernel<AT>, grid, dim3(128), 0, stream, (const AT*)x, ldx, W, logits, T, E, H));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// Ints of scratch the chunked sort needs for R routes over E experts.
long long ft_moe_sort_scratch(int R, int E) {
  return (long long)((R + SORT_CHUNK - 1) / SORT_CHUNK) * E;
}

// `scratch` (ft_moe_sort_scratch ints) selects the chunked sort; without it one
// warp per expert walks the routes (few routes: a decode batch).
int ft_moe_sort(const int* ids, int* counts, int* offsets, int* sorted_route, int* sorted_token,
                int* active, int* scratch, int R, int E, int k, cudaStream_t stream) {
  if (R <= 0) return FT_OK;
  if (scratch) {
    const int chunks = (R + SORT_CHUNK - 1) / SORT_CHUNK;
    const size_t hist = (size_t)E * sizeof(int), cur = 4 * hist;
    if (cur > 200 * 1024) return FT_ERR_SHAPE;
    if (cur > 48 * 1024) {
      cudaFuncSetAttribute(moe_chunk_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist);
      cudaFuncSetAttribute(moe_chunk_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cur);
    }
    moe_chunk_count_kernel<<<chunks, SORT_CHUNK, hist, stream>>>(ids, scratch, R, E);
    moe_chunk_scan_kernel<<<1, E < 1024 ? ((E + 31) / 32) * 32 : 1024, 0, stream>>>(scratch, counts, offsets,
                                                                                   active, chunks, E);
    moe_chunk_scatter_kernel<<<(chunks + 3) / 4, 128, cur, stream>>>(ids, scratch, offsets, sorted_route,
                                                                     sorted_token, R, E, k, chunks);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  const int warps = 4;
  const int blocks = (E + warps - 1) / warps;
  launch_pdl(moe_count_kernel, dim3(blocks), dim3(warps * 32), 0, stream, ids, counts, R, E);
  launch_pdl(moe_scatter_kernel, dim3(blocks), dim3(warps * 32), 0, stream, ids, (const int*)counts, offsets,
             sorted_route, sorted_token, active, R, E, k);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
