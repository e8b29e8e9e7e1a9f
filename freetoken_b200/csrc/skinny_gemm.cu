// C = A * W^T for FEW rows of A: the weight-streaming kernel of decode.
//
// Decode reads every weight it touches exactly once and does a handful of
// multiply-adds per weight, so the kernel is built around streaming W from HBM
// with many independent 16-byte loads in flight per warp.  The weight matrix is
// the M operand of mma.sync m16n8k16 (16 weight rows per warp tile), the tokens
// are the N operand (8 per MMA, NT MMAs side by side), accumulation is float32.
// A lane loads 8 consecutive bf16 of "its" weight row and the same 8 k-indices
// of "its" token; since a dot product does not care in which order k is
// visited, these 8 values are used as two k-pairs of two MMAs without any
// shuffle (the k-permutation is the same for both operands).
//
// A block is 4 warps that split K four ways over the same 16 weight rows and
// add their partial sums in warp order through shared memory, so a result does
// not depend on the launch shape.  Grouped use (experts): blockIdx.y is the
// j-th expert that has tokens (from the `active` list, so the grid is no larger
// than the number of routes), rows group_offsets[e]..group_offsets[e+1] of the
// sorted routes are its tokens, taken 8*NT at a time.
//
// Reference counterpart: python/freetoken/kernel/triton/decode_moe.py:5-75 (one
// program per route, CUDA-core FMAs: an expert's weights are read once per
// token that chose it); dense rows go through cuBLAS there
// (python/freetoken/layers/linear.py:31-32).
#include "common.cuh"

namespace ft {

struct SkinnyArgs {
  const __nv_bfloat16* A;
  const __nv_bfloat16* W;
  void* C;
  const int* group_offsets;  // [G+1] or nullptr
  const int* active;         // [G+1]: groups that have rows, then their number; or nullptr
  const int* a_rows;         // sorted row -> row of A, or nullptr
  const int* c_rows;         // sorted row -> row of C, or nullptr
  const float* row_scale;    // by row of C, or nullptr
  long long lda, ldc, w_group_stride;
  int M, N, K, G;
  int act;
  float act_alpha, act_limit;
};

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float glu_act_s(float g, float u, int act, float alpha, float limit) {
  if (act == 0) return (g / (1.f + __expf(-g))) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return (g / (1.f + __expf(-alpha * g))) * (u + 1.f);
}

// KS: warps per block, splitting K.  2 for the experts (gate_up bank: measured against 4
// warps, 26.3 instead of 29.8 us for the eight experts of a single token and level from
// batch 8 on; 1 and 8 are slower; down projection, rows of 1,536 values: two warps keep
// a warp's stream of a row twice as long and measured 3-5 % faster than four);
// 8 or 16 for dense matrices with few rows (QKV, O), where 4 warps per
// 16 weight rows would leave an SM with a handful of warps and too few loads in
// flight to fill the memory pipe.  KS is chosen from the weight's shape alone.
template <int NT, bool GLU, typename OT, int KS>
__global__ void __launch_bounds__(KS * 32) skinny_kernel(SkinnyArgs a) {
  constexpr int U = NT == 1 ? 4 : (NT == 2 ? 2 : 1);  // 32-k chunks in flight per warp
  constexpr int NG = GLU ? 2 : 1;
  __shared__ float red[KS][NT][NG][16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  pdl_wait();

  int group = blockIdx.y;
  if (a.active) {
    if ((int)blockIdx.y >= a.active[a.G]) return;
    group = a.active[blockIdx.y];
  }
  int row_begin = 0, row_end = a.M;
  if (a.group_offsets) {
    row_begin = a.group_offsets[group];
    row_end = a.group_offsets[group + 1];
  }
  if (row_end <= row_begin) return;
  const int n0 = blockIdx.x * 16;
  const __nv_bfloat16* W = a.W + (size_t)group * a.w_group_stride;
  const int K = a.K;
  // weight row pointers of this lane (rows beyond N are clamped and masked)
  const uint4* wrow[NG][2];
  bool wvalid[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = n0 + g + 8 * h;
    wvalid[h] = r < a.N;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const size_t rr = (size_t)(wvalid[h] ? r : 0) + (size_t)q * a.N;
      wrow[q][h] = reinterpret_cast<const uint4*>(W + rr * K);
    }
  }
  const int chunks = (K + 31) >> 5;
  const int per = (chunks + KS - 1) / KS;
  const int c_begin = warp * per, c_end = min(chunks, c_begin + per);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  for (int pass = row_begin; pass < row_end; pass += 8 * NT) {
    const uint4* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int row = pass + 8 * j + g;
      xrow[j] = nullptr;
      if (row < row_end) {
        const int src = a.a_rows ? a.a_rows[row] : row;
        xrow[j] = reinterpret_cast<const uint4*>(a.A + (size_t)src * a.lda);
      }
    }
    float acc[NG][NT][4];
#pragma unroll
    for (int q = 0; q < NG; ++q)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q][j][i] = 0.f;

    for (int c = c_begin; c < c_end; c += U) {
      uint4 wv[U][NG][2];
      uint4 xv[U][NT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k8 = ((c + u) << 2) + t;  // index in units of 8 elements
        const bool kin = (c + u) < c_end && (k8 << 3) < K;
#pragma unroll
        for (int q = 0; q < NG; ++q)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            wv[u][q][h] = (kin && wvalid[h]) ? ld_stream(wrow[q][h] + k8) : zero;
#pragma unroll
        for (int j = 0; j < NT; ++j)
          xv[u][j] = (kin && xrow[j]) ? __ldg(xrow[j] + k8) : zero;
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < NG; ++q)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma_bf16(acc[q][j], wv[u][q][0].x, wv[u][q][1].x, wv[u][q][0].y, wv[u][q][1].y,
                     xv[u][j].x, xv[u][j].y);
            mma_bf16(acc[q][j], wv[u][q][0].z, wv[u][q][1].z, wv[u][q][0].w, wv[u][q][1].w,
                     xv[u][j].z, xv[u][j].w);
          }
    }
#pragma unroll
    for (int q = 0; q < NG; ++q)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        red[warp][j][q][g][2 * t] = acc[q][j][0];
        red[warp][j][q][g][2 * t + 1] = acc[q][j][1];
        red[warp][j][q][g + 8][2 * t] = acc[q][j][2];
        red[warp][j][q][g + 8][2 * t + 1] = acc[q][j][3];
      }
    __syncthreads();
    OT* C = (OT*)a.C;
    for (int idx = threadIdx.x; idx < NT * 128; idx += KS * 32) {
      const int j = idx >> 7, tok = (idx & 127) >> 4, r = idx & 15;
      float s = 0.f, su = 0.f;
#pragma unroll
      for (int w = 0; w < KS; ++w) {
        s += red[w][j][0][r][tok];
        if (GLU) su += red[w][j][NG - 1][r][tok];
      }
      const int row = pass + 8 * j + tok, n = n0 + r;
      if (row < row_end && n < a.N) {
        const int crow = a.c_rows ? a.c_rows[row] : row;
        float v = GLU ? glu_act_s(s, su, a.act, a.act_alpha, a.act_limit) : s;
        if (a.row_scale) v *= a.row_scale[crow];
        C[(size_t)crow * a.ldc + n] = from_float<OT>(v);
      }
    }
    __syncthreads();
  }
}

template <bool GLU, typename OT, int KS>
int launch_nt(const SkinnyArgs& a, int nt, dim3 grid, cudaStream_t stream) {
  switch (nt) {
    case 1: launch_pdl(skinny_kernel<1, GLU, OT, KS>, grid, dim3(KS * 32), 0, stream, a); break;
    case 2: launch_pdl(skinny_kernel<2, GLU, OT, KS>, grid, dim3(KS * 32), 0, stream, a); break;
    case 4: launch_pdl(skinny_kernel<4, GLU, OT, KS>, grid, dim3(KS * 32), 0, stream, a); break;
    default: return FT_ERR_SHAPE;
  }
  return FT_OK;
}

// Warps per block for a dense [N, K] weight: 2 when there are blocks in plenty
// anyway (measured 4 % faster on the head), else doubled from 4 while the launch
// would hold fewer than about 1,500 warps and a warp keeps at least 8 chunks of
// 32 k.  Measured on a B200 at batch 1 / 8 (weights cold): QKV [8192 x 3072] 11.1 /
// 12.1 us with 4 warps (8: 12.5 / 13.9, 2: 14.4, 16: 15.5); O [3072 x 6144] 9.8 /
// 10.9 us with 8 warps (16: 11.6 / 12.1, 4: 14.7).  A function of the weight's shape
// only, so a token's result does not depend on what else is in the batch.
static int dense_k_split(int N, int K) {
  const long long tiles = (N + 15) / 16;
  const int chunks = (K + 31) / 32;
  int ks = 4;
  if (tiles * 2 >= 6000) return 2;      // blocks in plenty (the head): long streams per warp
  while (ks < 16 && tiles * ks < 1500 && chunks / (2 * ks) >= 8) ks *= 2;
  return ks;
}

}  // namespace ft

using namespace ft;

// A, W bfloat16; C bfloat16 or float32.  `rows_per_pass` in {8,16,32} picks
// how many tokens share one pass over the weights.  Needs K % 8 == 0,
// lda % 8 == 0 and 16-byte aligned base pointers; refuses anything else.
extern "C" int ft_skinny_gemm(const void* A, long long lda, const void* W,
                              long long w_group_stride, void* C, int c_dtype, long long ldc,
                              const int* group_offsets, const int* active, const int* a_rows,
                              const int* c_rows, const float* row_scale, int M, int N, int K, int G, int glu,
                              int act, float act_alpha, float act_limit, int rows_per_pass,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return FT_OK;
  if (K <= 0 || (K & 7) || (lda & 7) || G <= 0) return FT_ERR_SHAPE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((w_group_stride * 2) & 15)) return FT_ERR_SHAPE;
  if (G > 65535) return FT_ERR_SHAPE;
  SkinnyArgs a{(const __nv_bfloat16*)A, (const __nv_bfloat16*)W, C, group_offsets, active, a_rows,
               c_rows, row_scale, lda, ldc, w_group_stride, M, N, K, G, act, act_alpha, act_limit};
  // with the list of busy groups, no more groups than rows can have any
  dim3 grid((N + 15) / 16, active ? min(G, M) : G);
  const int nt = rows_per_pass / 8;
  int rc;
  int ks = (!glu && !group_offsets && G == 1) ? dense_k_split(N, K) : 4;
  // an expert's down projection has short rows: two warps a block keep a warp's stream
  // of a row long enough (a function of the weight's shape, like the dense choice)
  if (!glu && group_offsets && K <= 2048) ks = 2;
  if (c_dtype == FT_DTYPE_BF16) {
    if (glu) rc = launch_nt<true, __nv_bfloat16, 2>(a, nt, grid, stream);
    else if (ks == 2) rc = launch_nt<false, __nv_bfloat16, 2>(a, nt, grid, stream);
    else if (ks == 16) rc = launch_nt<false, __nv_bfloat16, 16>(a, nt, grid, stream);
    else if (ks == 8) rc = launch_nt<false, __nv_bfloat16, 8>(a, nt, grid, stream);
    else rc = launch_nt<false, __nv_bfloat16, 4>(a, nt, grid, stream);
  } else if (c_dtype == FT_DTYPE_F32) {
    if (glu) rc = launch_nt<true, float, 2>(a, nt, grid, stream);
    else if (ks == 2) rc = launch_nt<false, float, 2>(a, nt, grid, stream);
    else if (ks == 16) rc = launch_nt<false, float, 16>(a, nt, grid, stream);
    else if (ks == 8) rc = launch_nt<false, float, 8>(a, nt, grid, stream);
    else rc = launch_nt<false, float, 4>(a, nt, grid, stream);
  } else {
    return FT_ERR_DTYPE;
  }
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}
