// Decode attention: one query token per request against its paged keys.
//
// A CTA owns (token, KV head, key split).  The G query heads that share the KV
// head form the rows of a 16-row tensor-core tile (rows >= G are padding); the
// CTA's 4 warps each take 16 keys of every 64-key tile, keep a running
// max / sum / accumulator of their own in float32 and are merged at the end.
// K and V tiles go global -> shared with cp.async (16-byte chunks, three
// stages in flight), fragments are read with ldmatrix, products are
// mma.sync m16n8k16 bf16 with float32 accumulation; P is rounded to bf16
// before P*V as in the reference's tensor-core kernels.
// With splits > 1 every CTA writes an unnormalised partial (o, max, sum) and
// attn_merge combines the splits in ascending order.
//
// Reference: split-KV grouped decode in two stages,
// python/freetoken/kernel/triton/attention.py:147-349 (8 fixed splits; here the
// split count follows batch * kv_heads against the SM count), scale and mask
// :74,118-139.
#include "common.cuh"
#include "mma_utils.cuh"

namespace ft {

struct DecodeArgs {
  const __nv_bfloat16* q;    // [T, nq*d]
  __nv_bfloat16* out;        // [T, nq*d]
  float* part_o;             // [n_rows, nq, splits, d]
  float* part_ml;            // [n_rows, nq, splits, 2]
  const __nv_bfloat16* kv;   // [2, pages, nkv, P, d]
  const int* rows;           // token rows to process, or nullptr for 0..n_rows-1
  const int* token_pos;
  const int* token_seg;
  const int* block_table;
  long long page_stride, kv_stride;
  int nq, nkv, P, table_width, window;
  int n_rows, splits, split_keys;
  float scale;
};

constexpr int TILE = 64;    // keys per tile
constexpr int STAGES = 3;

template <int D>
__global__ void __launch_bounds__(128) attn_decode_kernel(DecodeArgs a) {
  constexpr int LD = D + 8;            // padded row: conflict-free ldmatrix
  constexpr int CH = D / 8;            // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [16][LD]
  __nv_bfloat16* sK = sQ + 16 * LD;                                       // [STAGES][TILE][LD]
  __nv_bfloat16* sV = sK + STAGES * TILE * LD;                            // [STAGES][TILE][LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_wait();

  const int G = a.nq / a.nkv;
  const int gtiles = (G + 15) / 16;
  const int kvh = blockIdx.y / gtiles, gt = blockIdx.y % gtiles;
  const int head0 = kvh * G + gt * 16;                 // first query head of this tile
  const int heads = min(16, G - gt * 16);
  const int row = blockIdx.x;
  const int tok = a.rows ? a.rows[row] : row;
  const int split = blockIdx.z;
  const int pos = a.token_pos[tok];
  const int* table = a.block_table + (size_t)a.token_seg[tok] * a.table_width;
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int k_begin = max(lo, split * a.split_keys) / TILE * TILE;
  const int k_end = min(pos + 1, (split + 1) * a.split_keys);
  const int first_valid = max(lo, split * a.split_keys);

  // Q tile -> shared (rows >= heads are zero)
  for (int idx = tid; idx < 16 * CH; idx += 128) {
    const int r = idx / CH, c = idx % CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < heads) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)tok * a.nq + head0 + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
  }

  const __nv_bfloat16* kbase = a.kv + (size_t)kvh * a.P * D;
  const __nv_bfloat16* vbase = kbase + a.kv_stride;
  const int ntiles = k_end > k_begin ? (k_end - k_begin + TILE - 1) / TILE : 0;

  // A tile lies inside one page when the page size is a multiple of the tile
  // (tiles start at multiples of 64): one table lookup per tile; otherwise every
  // key row looks its page up.
  const bool tile_in_page = (a.P % TILE) == 0;
  auto load_tile = [&](int tile, int stage) {
    const int j0 = k_begin + tile * TILE;
    __nv_bfloat16* dk = sK + stage * TILE * LD;
    __nv_bfloat16* dv = sV + stage * TILE * LD;
    if (tile_in_page) {
      const size_t page_off = (size_t)table[j0 / a.P] * a.page_stride + (size_t)(j0 % a.P) * D;
      const int last = pos - j0;                      // rows past the end repeat a valid key (masked later)
#pragma unroll
      for (int i = 0; i < TILE * CH / 128; ++i) {
        const int idx = tid + 128 * i;
        const int r = idx / CH, c = idx % CH;
        const size_t off = page_off + (size_t)min(r, last) * D + c * 8;
        cp_async16(dk + r * LD + c * 8, kbase + off);
        cp_async16(dv + r * LD + c * 8, vbase + off);
      }
      return;
    }
    for (int idx = tid; idx < TILE * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH;
      const int j = min(j0 + r, pos);               // rows past the end repeat a valid key (masked later)
      const size_t off = (size_t)table[j / a.P] * a.page_stride + (size_t)(j % a.P) * D + c * 8;
      cp_async16(dk + r * LD + c * 8, kbase + off);
      cp_async16(dv + r * LD + c * 8, vbase + off);
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < ntiles) load_tile(s, s);
    cp_async_commit();
  }
  __syncthreads();  // sQ visible

  // Q fragments for all k-steps
  unsigned qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int r = lane & 15, c = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(qf[ks], sQ + r * LD + c);
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g+8
  const float scale_log2 = a.scale * 1.4426950408889634f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int pre = tile + STAGES - 1;
    if (pre < ntiles) load_tile(pre, pre % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const int stage = tile % STAGES;
    const __nv_bfloat16* tk = sK + stage * TILE * LD + warp * 16 * LD;
    const __nv_bfloat16* tv = sV + stage * TILE * LD + warp * 16 * LD;
    const int j0 = k_begin + tile * TILE + warp * 16;    // first key of this warp's 16
    if (j0 <= pos && j0 + 15 >= first_valid) {
      float s[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        unsigned kf[4];
        // matrices: (keys 0-7,k 0-7) (keys 0-7,k 8-15) (keys 8-15,k 0-7) (keys 8-15,k 8-15)
        const int r = (lane & 7) + ((lane >> 4) << 3), c = ks * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(kf, tk + r * LD + c);
        mma16816(s[0], qf[ks], kf[0], kf[1]);
        mma16816(s[1], qf[ks], kf[2], kf[3]);
      }
      // mask, scale, running softmax (rows g and g+8; keys j0 + 8n + 2t4 + {0,1})
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = j0 + 8 * n + 2 * t4 + (i & 1);
          const bool ok = j <= pos && j >= first_valid && j < k_end;
          s[n][i] = ok ? s[n][i] * scale_log2 : -INFINITY;
          if (i < 2) mx0 = fmaxf(mx0, s[n][i]); else mx1 = fmaxf(mx1, s[n][i]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      // The running max only moves when it would grow by more than 2^8: below that
      // exp2(s - max) stays far inside float32 and bfloat16 range and the rescale of
      // the accumulator (64 multiplies a thread) is skipped.  The softmax is the same
      // function of the scores whichever offset is subtracted.
      const float mn0 = mx0 > m0 + 8.f ? mx0 : m0, mn1 = mx1 > m1 + 8.f ? mx1 : m1;
      const float al0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - mn0);
      const float al1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mn1);
      const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
      float sum0 = 0.f, sum1 = 0.f;
      unsigned pf[4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = fast_exp2(s[n][0] - base0), p1 = fast_exp2(s[n][1] - base0);
        const float p2 = fast_exp2(s[n][2] - base1), p3 = fast_exp2(s[n][3] - base1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pf[2 * n] = pack_bf16(p0, p1);
        pf[2 * n + 1] = pack_bf16(p2, p3);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * al0 + sum0;
      l1 = l1 * al1 + sum1;
      if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1)) {
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
          o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
        }
      }
      m0 = mn0;
      m1 = mn1;
      // A fragment of P for k16 = 16 keys: {tile0 rows g, tile0 rows g+8, tile1 rows g, tile1 rows g+8}
      const unsigned pa[4] = {pf[0], pf[1], pf[2], pf[3]};
#pragma unroll
      for (int nn = 0; nn < D / 16; ++nn) {
        unsigned vf[4];
        // V^T fragments for d columns nn*16 .. +15: trans matrices (keys 0-7, d 0-7),(keys 8-15, d 0-7),
        // (keys 0-7, d 8-15),(keys 8-15, d 8-15)
        const int r = (lane & 7) + (((lane >> 3) & 1) << 3), c = nn * 16 + (lane >> 4) * 8;
        ldsm_x4_t(vf, tv + r * LD + c);
        mma16816(o[2 * nn], pa, vf[0], vf[1]);
        mma16816(o[2 * nn + 1], pa, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps (each has rows g, g+8 with its own max / sum)
  float* red_o = reinterpret_cast<float*>(sK);          // [4][16][D]
  float* red_ml = red_o + 4 * 16 * D;                   // [4][16][2]
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int c = n * 8 + 2 * t4;
    red_o[(warp * 16 + g) * D + c] = o[n][0];
    red_o[(warp * 16 + g) * D + c + 1] = o[n][1];
    red_o[(warp * 16 + g + 8) * D + c] = o[n][2];
    red_o[(warp * 16 + g + 8) * D + c + 1] = o[n][3];
  }
  if (t4 == 0) {
    red_ml[(warp * 16 + g) * 2] = m0;
    red_ml[(warp * 16 + g) * 2 + 1] = l0;
    red_ml[(warp * 16 + g + 8) * 2] = m1;
    red_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
  }
  __syncthreads();
  for (int idx = tid; idx < heads * D; idx += 128) {
    const int r = idx / D, c = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, red_ml[(w * 16 + r) * 2]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_ml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
      l += red_ml[(w * 16 + r) * 2 + 1] * f;
      acc += red_o[(w * 16 + r) * D + c] * f;
    }
    const int head = head0 + r;
    if (a.splits == 1) {
      a.out[((size_t)tok * a.nq + head) * D + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t pi = ((size_t)row * a.nq + head) * a.splits + split;
      a.part_o[pi * D + c] = acc;
      if (c == 0) {
        a.part_ml[pi * 2] = m;        // log2 domain
        a.part_ml[pi * 2 + 1] = l;
      }
    }
  }
}

// out[tok, head, :] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), splits ascending.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, const int* __restrict__ rows,
                                  int nq, int d, int splits) {
  pdl_wait();

  const int row = blockIdx.x, head = blockIdx.y;
  const int tok = rows ? rows[row] : row;
  const size_t base = ((size_t)row * nq + head) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    l += (ms == -INFINITY) ? 0.f : part_ml[(base + s) * 2 + 1] * fast_exp2(ms - m);
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) acc += part_o[(base + s) * d + c] * fast_exp2(ms - m);
    }
    out[((size_t)tok * nq + head) * d + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  }
}

template <int D>
int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
  const int G = a.nq / a.nkv;
  const size_t smem = (size_t)(16 + 2 * STAGES * TILE) * (D + 8) * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.n_rows, a.nkv * ((G + 15) / 16), a.splits);
  launch_pdl(attn_decode_kernel<D>, grid, dim3(128), smem, stream, a);
  return FT_OK;
}

}  // namespace ft

using namespace ft;

// bfloat16 only; head_dim in {32, 64, 128}.  part_o / part_ml are needed when splits > 1.
extern "C" int ft_attn_decode(const void* q, void* out, float* part_o, float* part_ml,
                              const void* kv, const int* rows, const int* token_pos,
                              const int* token_seg, const int* block_table, long long page_stride,
                              long long kv_stride, int nq, int nkv, int d, int P, int table_width,
                              int window, int n_rows, int splits, int split_keys, float scale,
                              cudaStream_t stream) {
  if (n_rows <= 0) return FT_OK;
  if (nkv <= 0 || nq % nkv || splits < 1 || split_keys < TILE || split_keys % TILE) return FT_ERR_SHAPE;
  if (splits > 1 && (!part_o || !part_ml)) return FT_ERR_SHAPE;
  DecodeArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, part_o, part_ml,
               (const __nv_bfloat16*)kv, rows, token_pos, token_seg, block_table, page_stride,
               kv_stride, nq, nkv, P, table_width, window, n_rows, splits, split_keys, scale};
  int rc;
  switch (d) {
    case 32: rc = launch_decode<32>(a, stream); break;
    case 64: rc = launch_decode<64>(a, stream); break;
    case 128: rc = launch_decode<128>(a, stream); break;
    default: return FT_ERR_SHAPE;
  }
  if (rc != FT_OK) return rc;
  if (splits > 1) {
    dim3 grid(n_rows, nq);
    launch_pdl(attn_merge_kernel, grid, dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, rows, nq, d, splits);
  }
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// The split merge alone, for partials another kernel wrote in the same layout.
extern "C" int ft_attn_merge(const float* part_o, const float* part_ml, void* out, const int* rows,
                             int n_rows, int nq, int d, int splits, cudaStream_t stream) {
  if (n_rows <= 0 || splits < 1) return FT_OK;
  dim3 grid(n_rows, nq);
  launch_pdl(attn_merge_kernel, grid, dim3(128), 0, stream, part_o, part_ml, (__nv_bfloat16*)out, rows, nq, d,
             splits);
  FT_LAUNCH_CHECK();
  return FT_OK;
}
