// Prefill attention: the tokens of a prompt portion against the request's
// paged keys, the portion's own (just stored) keys included.
//
// A CTA owns (query tile of 64 tokens of one segment, query head); its 4 warps
// take 16 query rows each and walk the key tiles (64 keys) from the first
// visible key to the tile's diagonal.  K and V tiles go global -> shared with
// cp.async through the block table, two stages in flight; fragments come from
// ldmatrix, products are mma.sync m16n8k16 bf16 with float32 accumulation,
// the softmax state (max, sum) and the output accumulator are float32, P is
// rounded to bf16 before P*V.  Causal by absolute position; a window limits how
// far back a row looks.
//
// Reference: tiled extend kernel over cached prefix + fresh keys,
// python/freetoken/kernel/triton/attention.py:469-758 (tile 128x64, P cast to
// bf16 at :573); mask and scale :74,118-139.
#include "common.cuh"
#include "mma_utils.cuh"

namespace ft {

struct PrefillArgs {
  const __nv_bfloat16* q;    // [T, nq*d]
  __nv_bfloat16* out;        // [T, nq*d]
  const __nv_bfloat16* kv;   // [2, pages, nkv, P, d]
  const int* tile_seg;       // [tiles] segment of each query tile
  const int* tile_q0;        // [tiles] first token of the tile inside its segment
  const int* seg_q_start;    // [S+1]
  const int* seg_pos0;       // [S]
  const int* block_table;    // [S, table_width]
  long long page_stride, kv_stride;
  int nq, nkv, P, table_width, window;
  float scale;
};

constexpr int QT = 64;      // query rows per CTA
constexpr int KT = 64;      // keys per tile
constexpr int PSTAGES = 2;

template <int D>
__global__ void __launch_bounds__(128, 3) attn_prefill_kernel(PrefillArgs a) {
  constexpr int LD = D + 8;
  constexpr int CH = D / 8;
  static_assert(QT == KT, "the query tile borrows the second K stage");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [PSTAGES][KT][LD]
  __nv_bfloat16* sV = sK + PSTAGES * KT * LD;                        // [PSTAGES][KT][LD]
  // The query tile is only needed until its fragments sit in registers; it
  // borrows the second K stage, which the pipeline first fills after that.
  __nv_bfloat16* sQ = sK + KT * LD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  // the list is walked backwards: the tiles with the most keys start first
  const int tile_index = gridDim.x - 1 - blockIdx.x;
  const int seg = a.tile_seg[tile_index], q0 = a.tile_q0[tile_index];
  const int head = blockIdx.y;
  const int kvh = head / (a.nq / a.nkv);
  const int seg_begin = a.seg_q_start[seg];
  const int n = a.seg_q_start[seg + 1] - seg_begin;
  const int rows = min(QT, n - q0);
  const int tok0 = seg_begin + q0;              // first token row of the tile
  const int pos_first = a.seg_pos0[seg] + q0;   // position of the tile's first row
  const int pos_last = pos_first + rows - 1;
  const int* table = a.block_table + (size_t)seg * a.table_width;
  const int lo_tile = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int k_begin = lo_tile / KT * KT;
  const int ntiles = (pos_last - k_begin) / KT + 1;

  for (int idx = tid; idx < QT * CH; idx += 128) {
    const int r = idx / CH, c = idx % CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok0 + r) * a.nq + head) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
  }
  const __nv_bfloat16* kbase = a.kv + (size_t)kvh * a.P * D;
  const __nv_bfloat16* vbase = kbase + a.kv_stride;

  auto load_tile = [&](int tile, int stage) {
    const int j0 = k_begin + tile * KT;
    __nv_bfloat16* dk = sK + stage * KT * LD;
    __nv_bfloat16* dv = sV + stage * KT * LD;
    for (int idx = tid; idx < KT * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH;
      const int j = min(j0 + r, pos_last);        // rows past the end repeat a valid key (masked)
      const size_t off = (size_t)table[j / a.P] * a.page_stride + (size_t)(j % a.P) * D + c * 8;
      cp_async16(dk + r * LD + c * 8, kbase + off);
      cp_async16(dv + r * LD + c * 8, vbase + off);
    }
  };

  load_tile(0, 0);
  cp_async_commit();
  __syncthreads();

  unsigned qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int r = warp * 16 + (lane & 15), c = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(qf[ks], sQ + r * LD + c);
  }
  __syncthreads();      // every warp has its query fragments: the borrowed stage is free
  float o[D / 8][4];
#pragma unroll
  for (int nn = 0; nn < D / 8; ++nn)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nn][i] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float scale_log2 = a.scale * 1.4426950408889634f;
  const int pos_r0 = pos_first + warp * 16 + g, pos_r1 = pos_r0 + 8;   // this lane's two rows
  const int lo_r0 = a.window > 0 ? pos_r0 - a.window + 1 : 0;
  const int lo_r1 = a.window > 0 ? pos_r1 - a.window + 1 : 0;
  const int warp_pos_hi = pos_first + warp * 16 + 15;                  // last row of the warp
  const int warp_lo = a.window > 0 ? pos_first + warp * 16 - a.window + 1 : 0;

  for (int tile = 0; tile < ntiles; ++tile) {
    if (tile + 1 < ntiles) load_tile(tile + 1, (tile + 1) % PSTAGES);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int stage = tile % PSTAGES;
    const __nv_bfloat16* tk = sK + stage * KT * LD;
    const __nv_bfloat16* tv = sV + stage * KT * LD;
    const int j0 = k_begin + tile * KT;
    if (j0 <= warp_pos_hi && j0 + KT - 1 >= warp_lo) {
      float s[KT / 8][4];
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < KT / 16; ++np) {
          unsigned kf[4];
          const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3), c = ks * 16 + ((lane >> 3) & 1) * 8;
          ldsm_x4(kf, tk + r * LD + c);
          mma16816(s[2 * np], qf[ks], kf[0], kf[1]);
          mma16816(s[2 * np + 1], qf[ks], kf[2], kf[3]);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = j0 + 8 * nt + 2 * t4 + (i & 1);
          const bool ok = i < 2 ? (j <= pos_r0 && j >= lo_r0) : (j <= pos_r1 && j >= lo_r1);
          s[nt][i] = ok ? s[nt][i] * scale_log2 : -INFINITY;
          if (i < 2) mx0 = fmaxf(mx0, s[nt][i]); else mx1 = fmaxf(mx1, s[nt][i]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float al0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - mn0);
      const float al1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mn1);
      const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
      float sum0 = 0.f, sum1 = 0.f;
      unsigned pf[KT / 8][2];
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt) {
        const float p0 = fast_exp2(s[nt][0] - base0), p1 = fast_exp2(s[nt][1] - base0);
        const float p2 = fast_exp2(s[nt][2] - base1), p3 = fast_exp2(s[nt][3] - base1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pf[nt][0] = pack_bf16(p0, p1);
        pf[nt][1] = pack_bf16(p2, p3);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * al0 + sum0;
      l1 = l1 * al1 + sum1;
      m0 = mn0;
      m1 = mn1;
#pragma unroll
      for (int nn = 0; nn < D / 8; ++nn) {
        o[nn][0] *= al0; o[nn][1] *= al0; o[nn][2] *= al1; o[nn][3] *= al1;
      }
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        const unsigned pa[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
        for (int nn = 0; nn < D / 16; ++nn) {
          unsigned vf[4];
          const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), c = nn * 16 + (lane >> 4) * 8;
          ldsm_x4_t(vf, tv + r * LD + c);
          mma16816(o[2 * nn], pa, vf[0], vf[1]);
          mma16816(o[2 * nn + 1], pa, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int nn = 0; nn < D / 8; ++nn) {
    const int c = nn * 8 + 2 * t4;
    if (r0 < rows)
      *reinterpret_cast<unsigned*>(a.out + ((size_t)(tok0 + r0) * a.nq + head) * D + c) =
          pack_bf16(o[nn][0] * inv0, o[nn][1] * inv0);
    if (r1 < rows)
      *reinterpret_cast<unsigned*>(a.out + ((size_t)(tok0 + r1) * a.nq + head) * D + c) =
          pack_bf16(o[nn][2] * inv1, o[nn][3] * inv1);
  }
}

template <int D>
int launch_prefill(const PrefillArgs& a, int tiles, cudaStream_t stream) {
  const size_t smem = (size_t)(2 * PSTAGES * KT) * (D + 8) * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(tiles, a.nq);
  attn_prefill_kernel<D><<<grid, 128, smem, stream>>>(a);
  return FT_OK;
}

}  // namespace ft

using namespace ft;

// bfloat16 only; head_dim in {32, 64, 128}.  tile_seg / tile_q0 list the query
// tiles (64 tokens) of the segments to process.
extern "C" int ft_attn_prefill(const void* q, void* out, const void* kv, const int* tile_seg,
                               const int* tile_q0, const int* seg_q_start, const int* seg_pos0,
                               const int* block_table, long long page_stride, long long kv_stride,
                               int nq, int nkv, int d, int P, int table_width, int window,
                               int tiles, float scale, cudaStream_t stream) {
  if (tiles <= 0) return FT_OK;
  if (nkv <= 0 || nq % nkv) return FT_ERR_SHAPE;
  PrefillArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kv, tile_seg,
                tile_q0, seg_q_start, seg_pos0, block_table, page_stride, kv_stride, nq, nkv, P,
                table_width, window, scale};
  int rc;
  switch (d) {
    case 32: rc = launch_prefill<32>(a, tiles, stream); break;
    case 64: rc = launch_prefill<64>(a, tiles, stream); break;
    case 128: rc = launch_prefill<128>(a, tiles, stream); break;
    default: return FT_ERR_SHAPE;
  }
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}
