// C = A * W^T on CUDA cores in float32, dense or grouped by expert.
//
// This is the true 32-bit matrix path (no tensor cores, no reduced-precision
// mode) and the fallback for sizes the tensor-core kernels refuse.  Every
// output element is one thread's sum over k = 0..K-1 in ascending order, so a
// row's result does not depend on how many rows the launch holds, on the tile
// shape chosen, or on which expert group the row fell into.
//
// Grouped use (routed experts; reference python/freetoken/moe/fused.py:267-337,
// python/freetoken/kernel/triton/fused_moe.py:156-302): rows are sorted by
// expert, group_offsets[g]..group_offsets[g+1] are expert g's rows, W holds one
// [N,K] matrix per expert.  a_rows / c_rows redirect the input and output rows
// (token of a sorted route; route of a sorted row); row_scale multiplies the
// float32 accumulator before rounding (route weight, fused_moe.py:292-296).
// The SwiGLU epilogue reads W as [gate rows 0..N-1 ; up rows N..2N-1] and
// stores act(gate)*up (python/freetoken/kernel/triton/activation.py:96-107).
#include "common.cuh"

namespace ft {

struct GemmArgs {
  const void* A;
  const void* W;
  void* C;
  const int* group_offsets;  // [G+1] or nullptr (one group of M rows)
  const int* a_rows;         // [M] or nullptr
  const int* c_rows;         // [M] or nullptr
  const float* row_scale;    // indexed by output row, or nullptr
  long long lda, ldc, w_group_stride;
  int M, N, K, G;
  int act;  // 0 silu(g)*u, 1 swigluoai
  float act_alpha, act_limit;
};

__device__ __forceinline__ float glu_act(float g, float u, int act, float alpha, float limit) {
  if (act == 0) return (g / (1.f + expf(-g))) * u;
  // swigluoai: min(g,L) * sigmoid(alpha*min(g,L)) * (clamp(u,-L,L) + 1)
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return (g / (1.f + expf(-alpha * g))) * (u + 1.f);
}

constexpr int BN = 64;
constexpr int BK = 32;

template <typename AT, typename WT, typename OT, int BM, bool GLU>
__global__ void __launch_bounds__(256) gemm_rows_kernel(GemmArgs a) {
  constexpr int TM = BM / 16, TN = BN / 16;
  __shared__ float As[BM][BK + 1];
  __shared__ float Ws[BN][BK + 1];
  __shared__ float Us[GLU ? BN : 1][BK + 1];
  __shared__ int tile_info[3];  // group, first row, rows
  if (threadIdx.x == 0) {
    int group = 0, row0 = 0, rows = 0;
    if (!a.group_offsets) {
      row0 = blockIdx.x * BM;
      rows = min(BM, a.M - row0);
    } else {
      int tile = blockIdx.x;
      for (int g = 0; g < a.G; ++g) {
        const int begin = a.group_offsets[g], end = a.group_offsets[g + 1];
        const int nt = (end - begin + BM - 1) / BM;
        if (tile < nt) {
          group = g;
          row0 = begin + tile * BM;
          rows = min(BM, end - row0);
          break;
        }
        tile -= nt;
      }
    }
    tile_info[0] = group;
    tile_info[1] = row0;
    tile_info[2] = rows;
  }
  __syncthreads();
  const int group = tile_info[0], row0 = tile_info[1], rows = tile_info[2];
  if (rows <= 0) return;
  const int n0 = blockIdx.y * BN;
  const AT* A = (const AT*)a.A;
  const WT* W = (const WT*)a.W + (size_t)group * a.w_group_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  float acc[TM][TN], acu[GLU ? TM : 1][GLU ? TN : 1];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if (GLU) acu[i][j] = 0.f;
    }

  for (int k0 = 0; k0 < a.K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const int r = idx / BK, kk = idx % BK;
      float v = 0.f;
      if (r < rows && k0 + kk < a.K) {
        const int src = a.a_rows ? a.a_rows[row0 + r] : row0 + r;
        v = to_float(A[(size_t)src * a.lda + k0 + kk]);
      }
      As[r][kk] = v;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      const int n = idx / BK, kk = idx % BK;
      float v = 0.f, u = 0.f;
      if (n0 + n < a.N && k0 + kk < a.K) {
        v = to_float(W[(size_t)(n0 + n) * a.K + k0 + kk]);
        if (GLU) u = to_float(W[(size_t)(a.N + n0 + n) * a.K + k0 + kk]);
      }
      Ws[n][kk] = v;
      if (GLU) Us[n][kk] = u;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], wv[TN], uv[GLU ? TN : 1];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[ty + 16 * i][kk];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        wv[j] = Ws[tx + 16 * j][kk];
        if (GLU) uv[j] = Us[tx + 16 * j][kk];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if (GLU) acu[i][j] = fmaf(av[i], uv[j], acu[i][j]);
        }
    }
    __syncthreads();
  }

  OT* C = (OT*)a.C;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty + 16 * i;
    if (r >= rows) continue;
    const int crow = a.c_rows ? a.c_rows[row0 + r] : row0 + r;
    const float scale = a.row_scale ? a.row_scale[crow] : 1.f;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (GLU) v = glu_act(v, acu[i][j], a.act, a.act_alpha, a.act_limit);
      if (a.row_scale) v *= scale;
      C[(size_t)crow * a.ldc + n] = from_float<OT>(v);
    }
  }
}

// Dense product for many rows: the same arithmetic (every output element is
// one thread's fma chain over ascending k, so results are bit-identical to
// gemm_rows_kernel) with 16-byte global loads, k-major shared tiles and
// 128-bit shared loads.  Needs K % 32 == 0 and 16-byte aligned rows.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256) gemm_dense_kernel(GemmArgs a) {
  constexpr int TBM = 64, TBN = 64, TBK = 32;
  __shared__ __align__(16) float As[TBK][TBM + 4];
  __shared__ __align__(16) float Ws[TBK][TBN + 4];
  const int row0 = blockIdx.x * TBM, n0 = blockIdx.y * TBN;
  const AT* A = (const AT*)a.A;
  const WT* W = (const WT*)a.W;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 8;      // this thread loads row lr, k lk..lk+7
  const bool a_ok = row0 + lr < a.M, w_ok = n0 + lr < a.N;
  const AT* ap = A + (size_t)(a_ok ? row0 + lr : 0) * a.lda + lk;
  const WT* wp = W + (size_t)(w_ok ? n0 + lr : 0) * a.K + lk;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  float av[8], wv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) av[i] = wv[i] = 0.f;
  if (a_ok) load8(ap, av);
  if (w_ok) load8(wp, wv);
  for (int k0 = 0; k0 < a.K; k0 += TBK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      As[lk + i][lr] = av[i];
      Ws[lk + i][lr] = wv[i];
    }
    __syncthreads();
    if (k0 + TBK < a.K) {            // next tile's loads fly while this one is multiplied
      if (a_ok) load8(ap + k0 + TBK, av);
      if (w_ok) load8(wp + k0 + TBK, wv);
    }
#pragma unroll
    for (int kk = 0; kk < TBK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float ar[4] = {a4.x, a4.y, a4.z, a4.w}, wr[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
  OT* C = (OT*)a.C;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < a.N) C[(size_t)r * a.ldc + n] = from_float<OT>(acc[i][j]);
    }
  }
}

template <typename AT, typename WT, typename OT>
int launch(const GemmArgs& a, int glu, int max_tiles_hint, cudaStream_t stream) {
  const bool plain = !glu && !a.group_offsets && !a.a_rows && !a.c_rows && !a.row_scale;
  const int a_align = sizeof(AT) == 2 ? 7 : 3, w_align = sizeof(WT) == 2 ? 7 : 3;
  if (plain && a.M >= 64 && !(a.K & 31) && !(a.lda & a_align) && !(a.K & w_align) &&
      !((uintptr_t)a.A & 15) && !((uintptr_t)a.W & 15)) {
    dim3 grid((a.M + 63) / 64, (a.N + 63) / 64);
    gemm_dense_kernel<AT, WT, OT><<<grid, 256, 0, stream>>>(a);
    return FT_OK;
  }
  const int per_group = a.group_offsets ? a.M / max(a.G, 1) : a.M;
  const bool big = per_group >= 32;
  const int bm = big ? 64 : 16;
  const int tiles = (a.M + bm - 1) / bm + (a.group_offsets ? a.G : 0);
  dim3 grid(tiles, (a.N + BN - 1) / BN);
  (void)max_tiles_hint;
  if (big) {
    if (glu) gemm_rows_kernel<AT, WT, OT, 64, true><<<grid, 256, 0, stream>>>(a);
    else gemm_rows_kernel<AT, WT, OT, 64, false><<<grid, 256, 0, stream>>>(a);
  } else {
    if (glu) gemm_rows_kernel<AT, WT, OT, 16, true><<<grid, 256, 0, stream>>>(a);
    else gemm_rows_kernel<AT, WT, OT, 16, false><<<grid, 256, 0, stream>>>(a);
  }
  return FT_OK;
}

}  // namespace ft

using namespace ft;

// A, W, C element types are given by code; supported triples:
//   (f32,f32,f32) (f32,bf16,f32) (bf16,bf16,bf16) (bf16,bf16,f32) (bf16,f32,f32)
extern "C" int ft_gemm_rows(const void* A, int a_dtype, long long lda, const void* W, int w_dtype,
                            long long w_group_stride, void* C, int c_dtype, long long ldc,
                            const int* group_offsets, const int* a_rows, const int* c_rows,
                            const float* row_scale, int M, int N, int K, int G, int glu, int act,
                            float act_alpha, float act_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return FT_OK;
  if (K <= 0 || G <= 0) return FT_ERR_SHAPE;
  GemmArgs a{A, W, C, group_offsets, a_rows, c_rows, row_scale, lda, ldc, w_group_stride,
             M, N, K, G, act, act_alpha, act_limit};
  const int key = a_dtype * 100 + w_dtype * 10 + c_dtype;
  int rc;
  switch (key) {
    case 0: rc = launch<float, float, float>(a, glu, 0, stream); break;
    case 10: rc = launch<float, __nv_bfloat16, float>(a, glu, 0, stream); break;
    case 111: rc = launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(a, glu, 0, stream); break;
    case 110: rc = launch<__nv_bfloat16, __nv_bfloat16, float>(a, glu, 0, stream); break;
    case 100: rc = launch<__nv_bfloat16, float, float>(a, glu, 0, stream); break;
    default: return FT_ERR_DTYPE;
  }
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}
