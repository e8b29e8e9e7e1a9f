// Row-wise kernels: embedding gather, residual-add + RMSNorm, fused
// QK-norm + rotary + KV page store, top-k combine, row gather.
//
// All arithmetic is float32 whatever the storage type; one block owns one
// token, so a token's result does not depend on what else is in the launch.
//
// Formulas (reference file:line):
//   embedding row copy, no scale      python/freetoken/kernel/csrc/jit/index.cu:31-59
//   z=x+r; r<-z; y=z*rsqrt(mean(z^2)+eps)*w   python/freetoken/kernel/triton/norm.py:101-112
//   (1+w) form                        python/freetoken/kernel/triton/norm.py:69-72
//   per-layer QK norm over the whole projection
//                                     python/freetoken/models/minimax_m2/attention.py:45-47,78-79
//   per-head QK norm                  python/freetoken/models/minimax_m3/attention.py:54-56,90-91
//   NeoX / interleaved partial rotary python/freetoken/kernel/triton/rope.py:62-78
//   K,V rows stored after norm+rotary python/freetoken/kernel/csrc/jit/store.cu:25-53
//   sum over the k routes in float32  python/freetoken/kernel/triton/fused_moe.py:143-153
#include "common.cuh"

namespace ft {

// 4 consecutive elements as float32
__device__ __forceinline__ float4 load4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4f(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4f(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// ---------------------------------------------------------------- embedding
template <typename WT>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                                    float* __restrict__ residual, int H, int vocab) {
  pdl_wait();

  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // validated on the host; never index outside the table
  const WT* row = table + (size_t)id * H;
  float* out = residual + (size_t)t * H;
  // four elements a step where the row allows it (8-byte loads of bfloat16, 16-byte stores)
  if ((H & 3) == 0 && (((uintptr_t)table | (uintptr_t)residual) & 15) == 0 && (H * sizeof(WT)) % 16 == 0) {
    for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x)
      *reinterpret_cast<float4*>(out + 4 * i) = load4f(row + 4 * i);
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_float(row[i]);
}

// ------------------------------------------------------------------ rmsnorm
// residual (float32) is updated in place with delta when delta != nullptr.
// delta holds k rows per token (k > 1: the partial results of a token's k
// routes); they are added in ascending order in float32, then to the residual.
// A thread owns groups of 4 consecutive elements (element 4*(tid + j*blockDim));
// up to NORM_KEEP groups stay in registers between the two passes.
constexpr int NORM_THREADS = 512;
constexpr int NORM_KEEP = 4;

__device__ __forceinline__ void store4f(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// EAGER (a step of few tokens, where a launch is a chain of waits for L2 rather than a
// stream): the k partial rows of a piece are fetched four at a time before they are added,
// in the same order.  With every SM full of such blocks the extra loads in flight cost more
// than they save (25 -> 29 us at 2,048 tokens), so many tokens keep the one-by-one loop.
constexpr int ROW_KERNEL_EAGER_TOKENS = 64;   // up to this many tokens the row kernels fetch eagerly

template <typename AT, bool VEC, bool EAGER = false>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(const AT* __restrict__ delta, float* __restrict__ residual,
               const float* __restrict__ weight, AT* __restrict__ out, int H, float eps,
               int plus_one, int k) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  float* r = residual + (size_t)t * H;
  const AT* d = delta ? delta + (size_t)t * k * H : nullptr;
  AT* o = out + (size_t)t * H;
  const float one = plus_one ? 1.f : 0.f;
  float ss = 0.f;
  if (VEC) {
    float4 keep[NORM_KEEP];
    const int groups = H >> 2;
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
      const int gi = threadIdx.x + j * NORM_THREADS;
      if (gi < groups) {
        float4 z = load4f(r + 4 * gi);
        if (d) {
          float4 add = load4f(d + 4 * gi);
          if (EAGER) {
            for (int q0 = 1; q0 < k; q0 += 4) {
              float4 more[4];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                more[u] = q0 + u < k ? load4f(d + (size_t)(q0 + u) * H + 4 * gi) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (q0 + u < k) { add.x += more[u].x; add.y += more[u].y; add.z += more[u].z; add.w += more[u].w; }
            }
          } else {
            for (int q = 1; q < k; ++q) {
              const float4 more = load4f(d + (size_t)q * H + 4 * gi);
              add.x += more.x; add.y += more.y; add.z += more.z; add.w += more.w;
            }
          }
          z.x += add.x; z.y += add.y; z.z += add.z; z.w += add.w;
          store4f(r + 4 * gi, z);
        }
        keep[j] = z;
        ss += z.x * z.x;
        ss += z.y * z.y;
        ss += z.z * z.z;
        ss += z.w * z.w;
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_KEEP; ++j) {
      const int gi = threadIdx.x + j * NORM_THREADS;
      if (gi < groups) {
        const float4 w = load4f(weight + 4 * gi);
        const float4 z = keep[j];
        store4f(o + 4 * gi, make_float4(z.x * inv * (w.x + one), z.y * inv * (w.y + one),
                                        z.z * inv * (w.z + one), z.w * inv * (w.w + one)));
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float z = r[i];
    if (d) {
      float add = to_float(d[i]);
      for (int j = 1; j < k; ++j) add += to_float(d[(size_t)j * H + i]);
      z += add;
      r[i] = z;
    }
    ss += z * z;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    o[i] = from_float<AT>(r[i] * inv * (weight[i] + one));
  }
}

// ------------------------------------------------- qk-norm + rotary + store
struct QkRopeArgs {
  const void* qkv;        // [T, ld] rows: q (nq*d) | k (nkv*d) | v (nkv*d)
  void* q_out;            // [T, nq*d]
  void* kv_pages;         // [2, pages, nkv, P, d]; nullptr: this stop writes no cache
  const float* q_weight;  // per_layer: [nq*d]; per_head: [d]
  const float* k_weight;  // per_layer: [nkv*d]; per_head: [d]
  const float* cos_sin;   // [max_pos, R]: cos (R/2) | sin (R/2); nullptr or R=0: no rotation
  const int* token_pos;   // [T]
  const int* token_seg;   // [T]
  const int* block_table; // [S, table_width]
  long long ld;
  long long page_stride;  // elements between pages: nkv*P*d
  long long kv_stride;    // elements between the K and V halves
  int nq, nkv, d, R, P, table_width;
  int norm_mode;          // 0 none, 1 per layer, 2 per head
  int plus_one, interleaved;
  float eps;
};

template <typename AT>
__global__ void qk_rope_store_kernel(QkRopeArgs a) {
  pdl_wait();

  extern __shared__ float head_inv[];  // [nq + nkv] for per-head mode
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const AT* row = (const AT*)a.qkv + (size_t)t * a.ld;
  const int qn = a.nq * a.d, kn = a.nkv * a.d;
  const AT* q = row;
  const AT* k = row + qn;
  const AT* v = row + qn + kn;
  float inv_q = 1.f, inv_k = 1.f;
  if (a.norm_mode == 1) {
    float s = 0.f;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) { float x = to_float(q[i]); s += x * x; }
    inv_q = rsqrtf(block_sum(s, scratch) / (float)qn + a.eps);
    s = 0.f;
    for (int i = threadIdx.x; i < kn; i += blockDim.x) { float x = to_float(k[i]); s += x * x; }
    inv_k = rsqrtf(block_sum(s, scratch) / (float)kn + a.eps);
  } else if (a.norm_mode == 2) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < a.nq + a.nkv; h += nwarps) {
      const AT* hp = row + (size_t)h * a.d;  // q heads then k heads are contiguous
      float s = 0.f;
      for (int i = lane; i < a.d; i += 32) { float x = to_float(hp[i]); s += x * x; }
      s = warp_sum(s);
      if (lane == 0) head_inv[h] = rsqrtf(s / (float)a.d + a.eps);
    }
    __syncthreads();
  }
  const int pos = a.token_pos[t];
  const int half = a.R >> 1;
  const float* cs = (a.cos_sin && a.R > 0) ? a.cos_sin + (size_t)pos * a.R : nullptr;
  const float one = a.plus_one ? 1.f : 0.f;

  AT* qo = (AT*)a.q_out + (size_t)t * qn;
  AT* ko = nullptr;
  AT* vo = nullptr;
  if (a.kv_pages) {
    const int seg = a.token_seg[t];
    const int page = a.block_table[(size_t)seg * a.table_width + pos / a.P];
    const size_t base = (size_t)page * a.page_stride + (size_t)(pos % a.P) * a.d;
    ko = (AT*)a.kv_pages + base;
    vo = (AT*)a.kv_pages + a.kv_stride + base;
  }
  const size_t head_stride_cache = (size_t)a.P * a.d;

  // One work item = (head, i) for i < d - half: items with i < half rotate the
  // pair (i, i+half) [NeoX] or (2i, 2i+1) [interleaved]; the others pass one
  // element beyond the rotary span through.
  const int per_head = a.d - half;
  const int total_q = a.nq * per_head, total_k = a.nkv * per_head;
  for (int w = threadIdx.x; w < total_q + total_k; w += blockDim.x) {
    const bool is_q = w < total_q;
    const int ww = is_q ? w : w - total_q;
    const int h = ww / per_head, i = ww % per_head;
    const AT* src = (is_q ? q : k) + (size_t)h * a.d;
    const float* nw = is_q ? a.q_weight : a.k_weight;
    float inv = 1.f;
    if (a.norm_mode == 1) inv = is_q ? inv_q : inv_k;
    if (a.norm_mode == 2) inv = head_inv[is_q ? h : a.nq + h];
    AT* dst = is_q ? qo + (size_t)h * a.d : (ko ? ko + (size_t)h * head_stride_cache : nullptr);
    if (!dst) continue;
    if (i < half) {
      const int i0 = a.interleaved ? 2 * i : i;
      const int i1 = a.interleaved ? 2 * i + 1 : i + half;
      float x0 = to_float(src[i0]), x1 = to_float(src[i1]);
      if (a.norm_mode) {
        const int w0 = a.norm_mode == 1 ? h * a.d + i0 : i0;
        const int w1 = a.norm_mode == 1 ? h * a.d + i1 : i1;
        x0 = x0 * inv * (nw[w0] + one);
        x1 = x1 * inv * (nw[w1] + one);
      }
      float y0 = x0, y1 = x1;
      if (cs) {
        const float c = cs[i], s = cs[half + i];
        y0 = x0 * c - x1 * s;
        y1 = x1 * c + x0 * s;
      }
      dst[i0] = from_float<AT>(y0);
      dst[i1] = from_float<AT>(y1);
    } else {
      const int i0 = i + half;  // elements R .. d-1
      float x0 = to_float(src[i0]);
      if (a.norm_mode) {
        const int w0 = a.norm_mode == 1 ? h * a.d + i0 : i0;
        x0 = x0 * inv * (nw[w0] + one);
      }
      dst[i0] = from_float<AT>(x0);
    }
  }
  if (vo) {
    for (int w = threadIdx.x; w < kn; w += blockDim.x) {
      const int h = w / a.d, i = w % a.d;
      vo[(size_t)h * head_stride_cache + i] = v[w];
    }
  }
}

// Same work for bfloat16 rows in 16-byte pieces: head_dim % 8 == 0, NeoX
// pairing with rotary_dim % 16 == 0, so that a piece of 8 elements below R/2
// pairs with the piece R/2 further on.
struct Chunk8 { float v[8]; };
__device__ __forceinline__ Chunk8 unpack8(const uint4& raw) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  Chunk8 c;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    c.v[2 * i] = f.x;
    c.v[2 * i + 1] = f.y;
  }
  return c;
}
__device__ __forceinline__ Chunk8 load8(const __nv_bfloat16* p) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  Chunk8 c;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    c.v[2 * i] = f.x;
    c.v[2 * i + 1] = f.y;
  }
  return c;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Chunk8& c) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(c.v[2 * i], c.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ float sumsq8(const Chunk8& c) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += c.v[i] * c.v[i];
  return s;
}

// Sum of two values over the block in one round; every thread gets both.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch /* 66 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) { scratch[warp] = a; scratch[33 + warp] = b; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sa = 0.f, sb = 0.f;
    for (int w = 0; w < nwarps; ++w) { sa += scratch[w]; sb += scratch[33 + w]; }
    scratch[32] = sa;
    scratch[65] = sb;
  }
  __syncthreads();
  a = scratch[32];
  b = scratch[65];
}

// 8 consecutive floats (norm weights, cos / sin): two 16-byte loads when the
// address allows it
__device__ __forceinline__ void load8w(const float* p, float (&v)[8]) {
  if (((uintptr_t)p & 15) == 0) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = p[i];
  }
}

// 8 consecutive floats from a 16-byte aligned address
__device__ __forceinline__ void load8a(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// grid (tokens, parts): the blocks of a token split its heads between them;
// with the per-layer norm every block sums the whole q and k rows itself (a
// few KB from L2) so that no block waits for another.
// EAGER (few tokens): every input of a work item is fetched before any arithmetic, the
// norm weights, cos and sin without an alignment branch between them (the host checks their
// bases); with many tokens the registers that takes cost occupancy (33 -> 39 us at 2,048).
template <bool EAGER>
__global__ void __launch_bounds__(256) qk_rope_store_vec_kernel(QkRopeArgs a) {
  extern __shared__ float head_inv[];
  __shared__ float scratch[66];
  pdl_wait();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = (const __nv_bfloat16*)a.qkv + (size_t)t * a.ld;
  const int d = a.d, dc = d >> 3;                 // pieces per head
  const int qn = a.nq * d, kn = a.nkv * d;
  float inv_q = 1.f, inv_k = 1.f;
  if (a.norm_mode == 1) {
    // a thread's pieces four at a time: fetched together, summed in the same order as one by one
    float sq = 0.f, sk = 0.f;
    auto sum_pieces = [&](const __nv_bfloat16* base, int pieces, float& acc) {
      for (int c0 = threadIdx.x; c0 < pieces; c0 += 4 * blockDim.x) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * blockDim.x;
          raw[u] = c < pieces ? *reinterpret_cast<const uint4*>(base + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * (int)blockDim.x < pieces) acc += sumsq8(unpack8(raw[u]));
      }
    };
    sum_pieces(row, qn >> 3, sq);
    sum_pieces(row + qn, kn >> 3, sk);
    block_sum2(sq, sk, scratch);
    inv_q = rsqrtf(sq / (float)qn + a.eps);
    inv_k = rsqrtf(sk / (float)kn + a.eps);
  } else if (a.norm_mode == 2) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < a.nq + a.nkv; h += nwarps) {
      float s = 0.f;
      for (int c = lane; c < dc; c += 32) s += sumsq8(load8(row + (size_t)h * d + c * 8));
      s = warp_sum(s);
      if (lane == 0) head_inv[h] = rsqrtf(s / (float)d + a.eps);
    }
    __syncthreads();
  }
  const int pos = a.token_pos[t];
  const int half = a.R >> 1, hc = half >> 3;      // rotary half, in pieces
  const float* cs = (a.cos_sin && a.R > 0) ? a.cos_sin + (size_t)pos * a.R : nullptr;
  const float one = a.plus_one ? 1.f : 0.f;
  __nv_bfloat16* qo = (__nv_bfloat16*)a.q_out + (size_t)t * qn;
  __nv_bfloat16* ko = nullptr;
  __nv_bfloat16* vo = nullptr;
  if (a.kv_pages) {
    const int seg = a.token_seg[t];
    const int page = a.block_table[(size_t)seg * a.table_width + pos / a.P];
    const size_t base = (size_t)page * a.page_stride + (size_t)(pos % a.P) * d;
    ko = (__nv_bfloat16*)a.kv_pages + base;
    vo = (__nv_bfloat16*)a.kv_pages + a.kv_stride + base;
  }
  const size_t head_stride_cache = (size_t)a.P * d;
  const int per_head = dc - hc;                   // work items per head
  const int total_q = a.nq * per_head, total = total_q + a.nkv * per_head;
  // this block's share of the work items and of the V pieces
  const int parts = gridDim.y, part = blockIdx.y;
  const int w_begin = (int)((long long)total * part / parts), w_end = (int)((long long)total * (part + 1) / parts);
  for (int w = w_begin + threadIdx.x; w < w_end; w += blockDim.x) {
    const bool is_q = w < total_q;
    const int ww = is_q ? w : w - total_q;
    const int h = ww / per_head, ci = ww % per_head;
    if (!is_q && !ko) continue;
    const __nv_bfloat16* src = row + (is_q ? 0 : qn) + (size_t)h * d;
    __nv_bfloat16* dst = is_q ? qo + (size_t)h * d : ko + (size_t)h * head_stride_cache;
    const float* nw = is_q ? a.q_weight : a.k_weight;
    float inv = 1.f;
    if (a.norm_mode == 1) inv = is_q ? inv_q : inv_k;
    if (a.norm_mode == 2) inv = head_inv[is_q ? h : a.nq + h];
    const int wbase = a.norm_mode == 1 ? h * d : 0;
    if (EAGER) {
      if (ci < hc) {
        const int i0 = ci * 8, i1 = i0 + half;
        const uint4 r0 = *reinterpret_cast<const uint4*>(src + i0), r1 = *reinterpret_cast<const uint4*>(src + i1);
        float w0[8], w1[8], c[8], sn[8];
        if (a.norm_mode) {
          load8a(nw + wbase + i0, w0);
          load8a(nw + wbase + i1, w1);
        }
        if (cs) {
          load8a(cs + i0, c);
          load8a(cs + half + i0, sn);
        }
        Chunk8 x0 = unpack8(r0), x1 = unpack8(r1);
        if (a.norm_mode) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x0.v[i] = x0.v[i] * inv * (w0[i] + one);
            x1.v[i] = x1.v[i] * inv * (w1[i] + one);
          }
        }
        Chunk8 y0 = x0, y1 = x1;
        if (cs) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            y0.v[i] = x0.v[i] * c[i] - x1.v[i] * sn[i];
            y1.v[i] = x1.v[i] * c[i] + x0.v[i] * sn[i];
          }
        }
        store8(dst + i0, y0);
        store8(dst + i1, y1);
      } else {
        const int i0 = (ci + hc) * 8;               // pieces beyond the rotary span
        const uint4 r0 = *reinterpret_cast<const uint4*>(src + i0);
        float w0[8];
        if (a.norm_mode) load8a(nw + wbase + i0, w0);
        Chunk8 x0 = unpack8(r0);
        if (a.norm_mode) {
#pragma unroll
          for (int i = 0; i < 8; ++i) x0.v[i] = x0.v[i] * inv * (w0[i] + one);
        }
        store8(dst + i0, x0);
      }
      continue;
    }
    if (ci < hc) {
      const int i0 = ci * 8, i1 = i0 + half;
      Chunk8 x0 = load8(src + i0), x1 = load8(src + i1);
      if (a.norm_mode) {
        float w0[8], w1[8];
        load8w(nw + wbase + i0, w0);
        load8w(nw + wbase + i1, w1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x0.v[i] = x0.v[i] * inv * (w0[i] + one);
          x1.v[i] = x1.v[i] * inv * (w1[i] + one);
        }
      }
      Chunk8 y0 = x0, y1 = x1;
      if (cs) {
        float c[8], sn[8];
        load8w(cs + i0, c);
        load8w(cs + half + i0, sn);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          y0.v[i] = x0.v[i] * c[i] - x1.v[i] * sn[i];
          y1.v[i] = x1.v[i] * c[i] + x0.v[i] * sn[i];
        }
      }
      store8(dst + i0, y0);
      store8(dst + i1, y1);
    } else {
      const int i0 = (ci + hc) * 8;               // pieces beyond the rotary span
      Chunk8 x0 = load8(src + i0);
      if (a.norm_mode) {
        float w0[8];
        load8w(nw + wbase + i0, w0);
#pragma unroll
        for (int i = 0; i < 8; ++i) x0.v[i] = x0.v[i] * inv * (w0[i] + one);
      }
      store8(dst + i0, x0);
    }
  }
  if (vo) {
    const __nv_bfloat16* v = row + qn + kn;
    const int vc = kn >> 3;
    const int v_begin = (int)((long long)vc * part / parts), v_end = (int)((long long)vc * (part + 1) / parts);
    for (int c = v_begin + threadIdx.x; c < v_end; c += blockDim.x) {
      const int h = (c * 8) / d, i = (c * 8) % d;
      *reinterpret_cast<uint4*>(vo + (size_t)h * head_stride_cache + i) =
          *reinterpret_cast<const uint4*>(v + c * 8);
    }
  }
}

// --------------------------------------------------------------- top-k sum
// out[t,:] = sum_j parts[t*k+j,:] in float32, j ascending.
template <typename AT>
__global__ void combine_kernel(const AT* __restrict__ parts, AT* __restrict__ out, int k, int H) {
  pdl_wait();

  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < k; ++j) s += to_float(parts[((size_t)t * k + j) * H + i]);
    out[(size_t)t * H + i] = from_float<AT>(s);
  }
}

// ---------------------------------------------------------------- row gather
template <typename AT>
__global__ void gather_rows_kernel(const AT* __restrict__ src, const int* __restrict__ rows,
                                   AT* __restrict__ dst, int H) {
  pdl_wait();

  const int r = blockIdx.x;
  const AT* s = src + (size_t)rows[r] * H;
  AT* d = dst + (size_t)r * H;
  // 16 bytes per thread and step where rows allow it: element-wise stores of a 16-bit
  // type cost several times what their bytes would
  constexpr int PER = 16 / (int)sizeof(AT);
  if (H % PER == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(s);
    uint4* d4 = reinterpret_cast<uint4*>(d);
    for (int i = threadIdx.x; i < H / PER; i += blockDim.x) d4[i] = __ldg(s4 + i);
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = s[i];
}

// ------------------------------------------------------------ read stream
// Sums a buffer of 16-byte words: nothing but loads, eight in flight per thread.
// What a read-only stream reaches on this GPU - the ceiling of a decode step, which
// reads weights and cache and writes next to nothing (a copy, the usual yardstick,
// spends half of its traffic on writes).  partial[block] receives the block's sum.
__global__ void __launch_bounds__(256) read_sum_kernel(const uint4* __restrict__ src, long long n16,
                                                       unsigned* __restrict__ partial) {
  __shared__ unsigned red[256];
  unsigned acc = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 7 * stride < n16; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + i + u * stride));
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  for (; i < n16; i += stride) {
    const uint4 v = src[i];
    acc += v.x ^ v.y ^ v.z ^ v.w;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

// ids[rows[i]] = src[src_index[i]]: the tokens a step sampled become the next
// step's inputs without a round trip through the host.  An id outside the
// vocabulary (which the sampler never writes) becomes 0.
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ rows,
                                    const int* __restrict__ src, const int* __restrict__ src_index, int n,
                                    int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int t = src[src_index[i]];
  ids[rows[i]] = (t < 0 || t >= vocab) ? 0 : t;
}

}  // namespace ft

using namespace ft;

extern "C" {

int ft_patch_tokens(int* ids, const int* rows, const int* src, const int* src_index, int n, int vocab,
                    cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  ft::patch_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, rows, src, src_index, n, vocab);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_embed_gather(const int* ids, const void* table, int table_dtype, float* residual, int T,
                    int H, int vocab, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  FT_DISPATCH(table_dtype, WT,
              launch_pdl(embed_gather_kernel<WT>, dim3(T), dim3(256), 0, stream, ids, (const WT*)table, residual, H, vocab));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_rmsnorm(const void* delta, float* residual, const float* weight, void* out, int dtype,
               int T, int H, float eps, int plus_one, int k, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (k < 1) return FT_ERR_SHAPE;
  // 16-byte pieces when the row allows it and fits the registers kept between the passes
  const bool vec = !(H & 3) && H <= 4 * NORM_THREADS * NORM_KEEP && !((uintptr_t)delta & 15) &&
                   !((uintptr_t)residual & 15) && !((uintptr_t)weight & 15) && !((uintptr_t)out & 15);
  if (vec && T <= ROW_KERNEL_EAGER_TOKENS) {
    FT_DISPATCH(dtype, AT,
                (launch_pdl(rmsnorm_kernel<AT, true, true>, dim3(T), dim3(NORM_THREADS), 0, stream,
                            (const AT*)delta, residual, weight, (AT*)out, H, eps, plus_one, k)));
  } else if (vec) {
    FT_DISPATCH(dtype, AT,
                launch_pdl(rmsnorm_kernel<AT, true>, dim3(T), dim3(NORM_THREADS), 0, stream,
                           (const AT*)delta, residual, weight, (AT*)out, H, eps, plus_one, k));
  } else {
    FT_DISPATCH(dtype, AT,
                launch_pdl(rmsnorm_kernel<AT, false>, dim3(T), dim3(NORM_THREADS), 0, stream,
                           (const AT*)delta, residual, weight, (AT*)out, H, eps, plus_one, k));
  }
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_qk_rope_store(const void* qkv, void* q_out, void* kv_pages, const float* q_weight,
                     const float* k_weight, const float* cos_sin, const int* token_pos,
                     const int* token_seg, const int* block_table, long long ld,
                     long long page_stride, long long kv_stride, int nq, int nkv, int d, int R,
                     int P, int table_width, int norm_mode, int plus_one, int interleaved,
                     float eps, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (R < 0 || R > d || (R & 1) || norm_mode < 0 || norm_mode > 2) return FT_ERR_SHAPE;
  QkRopeArgs a{qkv, q_out, kv_pages, q_weight, k_weight, cos_sin, token_pos, token_seg,
               block_table, ld, page_stride, kv_stride, nq, nkv, d, R, P, table_width,
               norm_mode, plus_one, interleaved, eps};
  const size_t smem = (size_t)(nq + nkv) * sizeof(float);
  const bool aligned = !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) &&
                       !((uintptr_t)kv_pages & 15) && !(ld & 7) && !(page_stride & 7) &&
                       !(kv_stride & 7);
  if (dtype == FT_DTYPE_BF16 && aligned && !(d & 7) && !(R & 15) && !interleaved) {
    // few tokens: several blocks per token share its heads
    const int pieces = (nq + 2 * nkv) * (d >> 3);
    int parts = T >= 512 ? 1 : (pieces + 255) / 256;
    if (parts > 8) parts = 8;
    if (parts < 1) parts = 1;
    const bool eager = T <= ROW_KERNEL_EAGER_TOKENS && !((uintptr_t)q_weight & 15) && !((uintptr_t)k_weight & 15) &&
                       !((uintptr_t)cos_sin & 15);
    if (eager) launch_pdl(qk_rope_store_vec_kernel<true>, dim3(T, parts), dim3(256), smem, stream, a);
    else launch_pdl(qk_rope_store_vec_kernel<false>, dim3(T, parts), dim3(256), smem, stream, a);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  FT_DISPATCH(dtype, AT, launch_pdl(qk_rope_store_kernel<AT>, dim3(T), dim3(256), smem, stream, a));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_combine(const void* parts, void* out, int dtype, int T, int k, int H, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  FT_DISPATCH(dtype, AT, launch_pdl(combine_kernel<AT>, dim3(T), dim3(256), 0, stream, (const AT*)parts, (AT*)out, k, H));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// Reads `bytes` (a multiple of 16, 16-byte aligned) once; `partial` holds `blocks` words.
int ft_read_sum(const void* src, long long bytes, unsigned* partial, int blocks, cudaStream_t stream) {
  if (bytes <= 0 || blocks <= 0) return FT_OK;
  if ((bytes & 15) || ((uintptr_t)src & 15)) return FT_ERR_SHAPE;
  read_sum_kernel<<<blocks, 256, 0, stream>>>((const uint4*)src, bytes >> 4, partial);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_gather_rows(const void* src, const int* rows, void* dst, int dtype, int n, int H,
                   cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  FT_DISPATCH(dtype, AT,
              launch_pdl(gather_rows_kernel<AT>, dim3(n), dim3(128), 0, stream, (const AT*)src, rows, (AT*)dst, H));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
