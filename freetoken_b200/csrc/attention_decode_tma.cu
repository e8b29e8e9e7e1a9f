// Decode attention with K and V tiles fetched by TMA: the same arithmetic as
// attention_decode.cu (one query token per request, the G query heads of a KV
// head as rows of a 16-row mma.sync tile, 4 warps x 16 keys of every 64-key
// tile, float32 running max / sum / accumulator per warp, split-KV partials
// merged by attn_merge), with another way of feeding it:
//
//   warp 4     producer: per 64-key tile one TMA box per 64 head dims for K and for V
//              (5-D tensor map over the paged cache, page from the block table) into a
//              ring of three stages; completion on the stage's "full" mbarrier
//   warps 0-3  consumers: wait "full", ldmatrix from the 128-byte-swizzled tile,
//              mma.sync, and arrive on the stage's "empty" mbarrier - no block-wide
//              barrier inside the loop, no per-thread address arithmetic or cp.async
//
// With up to 8 splits the CTAs of a (row, KV head) form a thread-block CLUSTER along
// the split axis and merge among themselves: each leaves its partial result in its own
// shared memory, and after a cluster barrier every CTA reads its share of (head, dim)
// pairs from all of them through distributed shared memory, in split order - no partials
// in global memory and no merge kernel.  More splits than a cluster holds (long contexts)
// write partials for attn_merge as before.
//
// Needs head size 64 or 128 and a page size that is a multiple of 64 (a tile then
// lies inside one page); other shapes use attention_decode.cu.  Every mbarrier wait
// is bounded (about two seconds): on expiry the CTA writes a code into `status`
// and returns.
//
// Reference: split-KV grouped decode in two stages,
// python/freetoken/kernel/triton/attention.py:147-349; scale and mask :74,118-139.
#include <cooperative_groups.h>
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "mma_utils.cuh"
#include "tcgen05.cuh"

namespace ft {

struct DecodeTmaArgs {
  const __nv_bfloat16* q;    // [T, nq*d]
  __nv_bfloat16* out;        // [T, nq*d]
  float* part_o;             // [n_rows, nq, splits, d]
  float* part_ml;            // [n_rows, nq, splits, 2]
  const int* rows;           // token rows to process, or nullptr for 0..n_rows-1
  const int* token_pos;
  const int* token_seg;
  const int* block_table;
  int* status;
  int nq, nkv, P, table_width, window;
  int n_rows, splits, split_keys;
  float scale;
};

constexpr int DT_TILE = 64;
constexpr int DT_STAGES = 3;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int D, bool CLUSTER>
__global__ void __launch_bounds__(160) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_kv,
                                                              DecodeTmaArgs a) {
  constexpr int TILE = DT_TILE, STAGES = DT_STAGES;
  constexpr int NB = D / 64;                    // 64-wide (128-byte) blocks per head
  constexpr int KB = TILE * 128;                // bytes of one block of K or V
  constexpr int STAGE = 2 * NB * KB;            // K blocks, then V blocks
  constexpr int LD = D + 8;
  constexpr int CH = D / 8;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* stages = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(stages + STAGES * STAGE);     // [16][LD]
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ volatile int gave_up;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  if (tid == 0) {
    gave_up = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
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
  const int ntiles = k_end > k_begin ? (k_end - k_begin + TILE - 1) / TILE : 0;

  // Q tile -> shared (rows >= heads are zero), by the consumers
  if (warp < 4) {
    for (int idx = tid; idx < 16 * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < heads) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)tok * a.nq + head0 + r) * D + c * 8);
      *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
    }
  }
  __syncthreads();   // barriers initialised, sQ visible

  if (warp == 4) {
    if (lane == 0) {
      int issued = 0;
      for (int tile = 0; tile < ntiles; ++tile, ++issued) {
        const int s = tile % STAGES;
        if (!mbar_wait(&empty_bar[s], (((unsigned)(tile / STAGES)) & 1u) ^ 1u, &gave_up)) {
          atomicCAS(a.status, 0, FT_ST_DECODE_PRODUCER);
          gave_up = 1;
          break;
        }
        const int j0 = k_begin + tile * TILE;
        const int page = table[j0 / a.P], off = j0 % a.P;
        unsigned char* st = stages + s * STAGE;
        mbar_expect_tx(&full_bar[s], STAGE);
#pragma unroll
        for (int h = 0; h < NB; ++h) {
          tma_load_5d(st + h * KB, &tm_kv, h * 64, off, kvh, page, 0, &full_bar[s]);
          tma_load_5d(st + (NB + h) * KB, &tm_kv, h * 64, off, kvh, page, 1, &full_bar[s]);
        }
      }
      if (gave_up) {
        // let copies already in flight land before the CTA (and its shared memory) goes away
        for (int tile = issued > STAGES ? issued - STAGES : 0; tile < issued; ++tile) {
          const unsigned long long t0 = global_ns();
          while (!mbar_try(&full_bar[tile % STAGES], ((unsigned)(tile / STAGES)) & 1u) &&
                 global_ns() - t0 < 100000000ull) {}
        }
      }
    }
    if (CLUSTER) {
      // stay for the cluster's two barriers: the others read this CTA's shared memory
      cooperative_groups::this_cluster().sync();
      cooperative_groups::this_cluster().sync();
    }
    return;
  }

  // ---- consumers -------------------------------------------------------------------
  // byte offset of 16-byte chunk `c16` of key row `r` inside a K (or V) tile
  auto sw_off = [](int r, int c16) -> int {
    return (c16 >> 3) * KB + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
  };
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
    const int stage = tile % STAGES;
    bool ok = mbar_wait(&full_bar[stage], ((unsigned)(tile / STAGES)) & 1u, &gave_up);
    if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_DECODE_CONSUMER); gave_up = 1; }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) break;
    const unsigned char* tk = stages + stage * STAGE;
    const unsigned char* tv = tk + NB * KB;
    const int j0 = k_begin + tile * TILE + warp * 16;    // first key of this warp's 16
    if (j0 <= pos && j0 + 15 >= first_valid) {
      if (j0 + 15 > pos) {
        // Keys past the request's last one: the box brought whatever the page held
        // before.  Their scores are masked, but 0 * V must stay 0 even if an earlier
        // request left a NaN or an infinity there: those V rows are zeroed.
        unsigned char* vrows = const_cast<unsigned char*>(tv);
        for (int idx = lane; idx < 16 * CH; idx += 32) {
          const int r = idx / CH, c16 = idx % CH;
          if (j0 + r > pos) *reinterpret_cast<uint4*>(vrows + sw_off(warp * 16 + r, c16)) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
        __syncwarp();
      }
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
        ldsm_x4(kf, tk + sw_off(warp * 16 + r, c >> 3));
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
        ldsm_x4_t(vf, tv + sw_off(warp * 16 + r, c >> 3));
        mma16816(o[2 * nn], pa, vf[0], vf[1]);
        mma16816(o[2 * nn + 1], pa, vf[2], vf[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
  }
  consumer_sync();   // every consumer is done with the stages: their memory holds the merge now

  // merge the four warps (each has rows g, g+8 with its own max / sum)
  float* red_o = reinterpret_cast<float*>(stages);          // [4][16][D]
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
  consumer_sync();
  // this CTA's result per (head row, dim): unnormalised sum, max (log2 domain) and weight sum
  float* xo = red_ml + 4 * 16 * 2;                      // [16][D]   (cluster exchange)
  float* xml = xo + 16 * D;                             // [16][2]
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
    if (CLUSTER) {
      xo[r * D + c] = acc;
      if (c == 0) {
        xml[r * 2] = m;
        xml[r * 2 + 1] = l;
      }
    } else if (a.splits == 1) {
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
  if (CLUSTER) {
    // out[head, c] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), splits ascending; the
    // (head, dim) pairs are dealt out over the cluster's CTAs, each reads every CTA's share
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int nsplit = a.splits, me = split;            // cluster = the splits of this (row, head tile)
    const int total = heads * D;
    const int share = (total + nsplit - 1) / nsplit;
    for (int idx = me * share + tid; idx < min(total, (me + 1) * share); idx += 128) {
      const int r = idx / D, c = idx % D;
      float m = -INFINITY;
      for (int s2 = 0; s2 < nsplit; ++s2) m = fmaxf(m, cluster.map_shared_rank(xml, s2)[r * 2]);
      float l = 0.f, acc = 0.f;
      for (int s2 = 0; s2 < nsplit; ++s2) {
        const float* rml = cluster.map_shared_rank(xml, s2);
        const float ms = rml[r * 2];
        if (ms != -INFINITY) {
          const float f = fast_exp2(ms - m);
          l += rml[r * 2 + 1] * f;
          acc += cluster.map_shared_rank(xo, s2)[r * D + c] * f;
        }
      }
      a.out[((size_t)tok * a.nq + head0 + r) * D + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
    cluster.sync();        // nobody leaves while its shared memory may still be read
  }
}


constexpr int DT_MAX_CLUSTER = 8;      // portable cluster size

template <int D>
int launch_decode_tma(const CUtensorMap& mkv, const DecodeTmaArgs& a, cudaStream_t stream) {
  const int G = a.nq / a.nkv;
  const size_t smem = (size_t)DT_STAGES * 2 * (D / 64) * DT_TILE * 128 + 16 * (D + 8) * sizeof(__nv_bfloat16) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.n_rows, a.nkv * ((G + 15) / 16), a.splits);
  if (a.splits > 1 && a.splits <= DT_MAX_CLUSTER && !a.part_o) {
    // the splits of a (row, head tile) as one cluster along z
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(160);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = (unsigned)a.splits;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_tma_kernel<D, true>, mkv, a);
    return e == cudaSuccess ? FT_OK : (int)e;
  }
  launch_pdl(attn_decode_tma_kernel<D, false>, grid, dim3(160), smem, stream, mkv, a);
  return FT_OK;
}

}  // namespace ft

using namespace ft;

// bfloat16; head_dim 64 or 128; page size a multiple of 64.  `map_kv`: the 5-D map
// over the layer's pages (ft_attn_tc_kv_map of the prefill library).  Up to 8 splits
// are merged inside the kernel by a cluster when part_o is null; otherwise part_o /
// part_ml receive the partials and the caller merges them with ft_attn_merge.
extern "C" int ft_attn_decode_tma(const void* map_kv, const void* q, void* out, float* part_o,
                                  float* part_ml, const int* rows, const int* token_pos,
                                  const int* token_seg, const int* block_table, int* status, int nq,
                                  int nkv, int d, int P, int table_width, int window, int n_rows,
                                  int splits, int split_keys, float scale, cudaStream_t stream) {
  if (n_rows <= 0) return FT_OK;
  if (nkv <= 0 || nq % nkv || splits < 1 || split_keys < DT_TILE || split_keys % DT_TILE || P % DT_TILE)
    return FT_ERR_SHAPE;
  if (splits > DT_MAX_CLUSTER && (!part_o || !part_ml)) return FT_ERR_SHAPE;
  CUtensorMap mkv;
  memcpy(&mkv, map_kv, sizeof(mkv));
  DecodeTmaArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, part_o, part_ml, rows, token_pos,
                  token_seg, block_table, status, nq, nkv, P, table_width, window, n_rows, splits,
                  split_keys, scale};
  int rc;
  switch (d) {
    case 64: rc = launch_decode_tma<64>(mkv, a, stream); break;
    case 128: rc = launch_decode_tma<128>(mkv, a, stream); break;
    default: return FT_ERR_SHAPE;
  }
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}
