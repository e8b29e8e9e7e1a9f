// Causal GQA softmax attention over the paged cache on CUDA cores.
//
// One warp owns one (token, query head).  It walks the keys in chunks of 32
// that are aligned to absolute positions (chunk c = keys 32c..32c+31), keeps a
// running max / sum / accumulator in float32 and visits keys in ascending
// order inside each chunk.  The arithmetic for a (token, head) therefore does
// not depend on whether the token came in a long prompt portion, a two-token
// portion or alone as a decode token, nor on which pages hold the keys.  This
// is the float32 path's attention and the fallback for head sizes the
// tensor-core kernels refuse.
//
// Formula (python/freetoken/kernel/triton/attention.py:74,118-139): scores
// q.k * scale for keys j <= pos (and j > pos - window when a window is set),
// softmax over them, weighted sum of v; query head h reads KV head h / group.
#include "common.cuh"

namespace ft {

struct AttnArgs {
  const void* q;          // [T, nq*d]
  void* out;              // [T, nq*d]
  const void* kv_pages;   // [2, pages, nkv, P, d]
  const int* token_pos;   // [T]
  const int* token_seg;   // [T]
  const int* block_table; // [S, table_width]
  const int* rows;        // token rows to process, or nullptr for 0..T-1
  long long page_stride, kv_stride;
  int nq, nkv, d, P, table_width, window;  // window <= 0: none
  float scale;
};

template <typename AT, bool EXACT>
__global__ void __launch_bounds__(128) attn_paged_kernel(AttnArgs a) {
  extern __shared__ float qs[];  // [4 warps][d]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = a.rows ? a.rows[blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y * 4 + warp;
  if (h >= a.nq) return;
  const int kvh = h / (a.nq / a.nkv);
  const int d = a.d;
  float* qv = qs + warp * d;
  const AT* q = (const AT*)a.q + ((size_t)t * a.nq + h) * d;
  for (int i = lane; i < d; i += 32) qv[i] = to_float(q[i]);
  __syncwarp();

  const int pos = a.token_pos[t];
  const int* table = a.block_table + (size_t)a.token_seg[t] * a.table_width;
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const AT* kbase = (const AT*)a.kv_pages + (size_t)kvh * a.P * d;
  const AT* vbase = kbase + a.kv_stride;

  constexpr int MAXD = 8;  // output dims per lane: head sizes up to 256
  float acc[MAXD];
#pragma unroll
  for (int c = 0; c < MAXD; ++c) acc[c] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c0 = (lo / 32) * 32; c0 <= pos; c0 += 32) {
    const int j = c0 + lane;
    const bool valid = j >= lo && j <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / a.P];
      const AT* kr = kbase + (size_t)page * a.page_stride + (size_t)(j % a.P) * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qv[i], to_float(kr[i]), dot);
      s = dot * a.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? (EXACT ? expf(s - m_new) : __expf(s - m_new)) : 0.f;
    const float alpha = (m == -INFINITY) ? 0.f : (EXACT ? expf(m - m_new) : __expf(m - m_new));
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < MAXD; ++c) acc[c] *= alpha;
    const int jj_lo = max(lo - c0, 0), jj_hi = min(pos - c0, 31);
    for (int jj = jj_lo; jj <= jj_hi; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int jk = c0 + jj;
      const int page = table[jk / a.P];
      const AT* vr = vbase + (size_t)page * a.page_stride + (size_t)(jk % a.P) * d;
#pragma unroll
      for (int c = 0; c < MAXD; ++c) {
        const int i = lane + 32 * c;
        if (i < d) acc[c] = fmaf(pj, to_float(vr[i]), acc[c]);
      }
    }
  }
  AT* o = (AT*)a.out + ((size_t)t * a.nq + h) * d;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < MAXD; ++c) {
    const int i = lane + 32 * c;
    if (i < d) o[i] = from_float<AT>(acc[c] * inv);
  }
}

}  // namespace ft

using namespace ft;

extern "C" int ft_attn_paged_simt(const void* q, void* out, const void* kv_pages,
                                  const int* token_pos, const int* token_seg,
                                  const int* block_table, const int* rows,
                                  long long page_stride, long long kv_stride, int nq, int nkv, int d, int P,
                                  int table_width, int window, float scale, int dtype, int T,
                                  cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (d > 256 || d <= 0 || nkv <= 0 || nq % nkv) return FT_ERR_SHAPE;
  AttnArgs a{q, out, kv_pages, token_pos, token_seg, block_table, rows, page_stride, kv_stride,
             nq, nkv, d, P, table_width, window, scale};
  dim3 grid(T, (nq + 3) / 4);
  const size_t smem = 4 * (size_t)d * sizeof(float);
  if (dtype == FT_DTYPE_F32) attn_paged_kernel<float, true><<<grid, 128, smem, stream>>>(a);
  else if (dtype == FT_DTYPE_BF16) attn_paged_kernel<__nv_bfloat16, false><<<grid, 128, smem, stream>>>(a);
  else return FT_ERR_DTYPE;
  FT_LAUNCH_CHECK();
  return FT_OK;
}
