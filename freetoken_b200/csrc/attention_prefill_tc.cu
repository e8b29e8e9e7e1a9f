// Prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), K and
// V pages brought in by TMA straight from the paged cache.
//
// A CTA owns 128 query tokens of one segment and one query head and walks the
// key tiles (64 keys, one TMA box per 64 head dims, through the block table)
// from key 0 to the tile's diagonal:
//
//   S[128 q, 64 keys]  = Q K^T      tcgen05.mma, Q and K both K-major from shared
//                                    memory, accumulator in TMEM
//   softmax            : a thread owns one query row (one TMEM lane): tcgen05.ld
//                        the row, scale, mask by absolute position, running max
//                        and sum in float32, P rounded to bfloat16 and written
//                        back over S in TMEM (two keys per 32-bit column)
//   O[128 q, d]       += P V        tcgen05.mma, P from TMEM, V MN-major from shared
//                                    memory (the cache keeps keys as rows),
//                                    accumulator in TMEM; when a row's max grows
//                                    the softmax threads rescale O in TMEM first
//
//   warp 0     TMA producer (Q once; K and V tiles into rings of two stages each)
//   warp 1     TMEM allocation; one thread issues the MMAs and commits
//   warps 2-5  softmax and the final normalise + store
// S has two TMEM buffers: the S product of tile j+1 is issued before the O
// product of tile j, so it runs under the softmax of tile j.  Two CTAs fit an SM
// (96 KB of shared memory and 256 TMEM columns each at head size 128).
//
// Every mbarrier wait is bounded (about two seconds): on expiry the CTA writes
// a code into `status`, stops issuing work, frees its TMEM and returns.
//
// Reference: tiled extend kernel over cached prefix + fresh keys,
// python/freetoken/kernel/triton/attention.py:469-758 (tile 128x64, P cast to
// bf16 at :573); mask and scale :74,118-139.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "mma_utils.cuh"
#include "tcgen05.cuh"

namespace ft {

constexpr int AQ = 128;    // query rows per CTA (UMMA M)
constexpr int AK = 64;     // keys per tile (UMMA N of S, K extent of P V)

struct PrefillTcArgs {
  __nv_bfloat16* out;        // [T, nq*d]
  const int* tile_seg;       // [tiles] segment of each 64-token query tile
  const int* tile_q0;        // [tiles] first token of the tile inside its segment
  const int* seg_q_start;    // [S+1]
  const int* seg_pos0;       // [S]
  const int* block_table;    // [S, table_width]
  int* status;
  int nq, nkv, P, table_width;
  float scale_log2;          // sm_scale * log2(e)
};

// HPC: query heads per CTA.  1: the CTA's 128 rows are 128 tokens of one head.
// 2: they are 64 tokens of two heads that share a KV head (an even group size):
// the K and V tiles a CTA fetches then serve two heads, which halves the
// L2 -> shared memory traffic per product, the scarcer resource at this tile size.
template <int D, int HPC>
__global__ void __launch_bounds__(192, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                 const __grid_constant__ CUtensorMap tm_q2,
                                                                 const __grid_constant__ CUtensorMap tm_kv,
                                                                 PrefillTcArgs a) {
  constexpr int NB = D / 64;                 // 64-wide (128-byte) blocks per head
  constexpr int QB = AQ * 128;               // bytes of one block of Q
  constexpr int KB = AK * 128;               // bytes of one block of K or V
  constexpr int Q_BYTES = NB * QB, K_BYTES = NB * KB;
  constexpr unsigned TMEM_COLS = 256u;       // O: D columns, then S/P: 2 x 64

  // the host lists 64-token tiles; a CTA takes an even one together with its successor
  const int tile_index = gridDim.x - 1 - blockIdx.x;     // backwards: most keys first
  constexpr int TOK = AQ / HPC;                       // tokens per CTA
  const int q0 = a.tile_q0[tile_index];
  if (q0 % TOK) return;                               // HPC == 1: a CTA takes an even list tile and its successor
  const int seg = a.tile_seg[tile_index];

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* sQ = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* sKr = sQ + Q_BYTES;                       // K ring [2]
  unsigned char* sVr = sKr + 2 * K_BYTES;                  // V ring [2]
  __shared__ __align__(8) unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2],
      p_full[2], pv_done, v_clean;
  __shared__ unsigned tmem_slot;
  __shared__ volatile int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * HPC;                  // first of the CTA's heads (same KV head: G % HPC == 0)
  const int kvh = head / (a.nq / a.nkv);
  const int seg_begin = a.seg_q_start[seg];
  const int n = a.seg_q_start[seg + 1] - seg_begin;
  const int rows = min(TOK, n - q0);                  // tokens this CTA really has
  const int tok0 = seg_begin + q0;
  const int pos_first = a.seg_pos0[seg] + q0;
  const int ntiles = (pos_first + rows - 1) / AK + 1;
  // keys of the last tile past the segment's last token: whatever the page held before
  const int stale_from = pos_first + rows - (ntiles - 1) * AK;      // first such key row, AK if none

  if (threadIdx.x == 0) {
    gave_up = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4);
    }
    mbar_init(&pv_done, 1);
    mbar_init(&v_clean, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  const unsigned tmem_o = tmem_base, tmem_s = tmem_base + D;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
      for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int hh = 0; hh < HPC; ++hh)      // head hh fills rows hh*TOK .. of every 64-wide block
          tma_load_2d(sQ + h * QB + hh * TOK * 128, HPC == 1 ? &tm_q : &tm_q2, (head + hh) * D + h * 64, tok0,
                      &q_full);
      const int* table = a.block_table + (size_t)seg * a.table_width;
      // K runs one tile ahead of V: K_j is wanted a whole softmax earlier than V_j
      int k_issued = 0, v_issued = 0;
      for (int j = 0; j <= ntiles; ++j) {
        if (j < ntiles) {
          const int s = j & 1;
          if (!mbar_wait(&k_empty[s], (((unsigned)j >> 1) & 1u) ^ 1u, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_PREFILL_PRODUCER);
            gave_up = 1;
            break;
          }
          const int key0 = j * AK;
          const int page = table[key0 / a.P], off = key0 % a.P;
          mbar_expect_tx(&k_full[s], K_BYTES);
#pragma unroll
          for (int h = 0; h < NB; ++h)
            tma_load_5d(sKr + s * K_BYTES + h * KB, &tm_kv, h * 64, off, kvh, page, 0, &k_full[s]);
          ++k_issued;
        }
        if (j > 0) {
          const int i = j - 1, s = i & 1;
          if (!mbar_wait(&v_empty[s], (((unsigned)i >> 1) & 1u) ^ 1u, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_PREFILL_PRODUCER);
            gave_up = 1;
            break;
          }
          const int key0 = i * AK;
          const int page = table[key0 / a.P], off = key0 % a.P;
          mbar_expect_tx(&v_full[s], K_BYTES);
#pragma unroll
          for (int h = 0; h < NB; ++h)
            tma_load_5d(sVr + s * K_BYTES + h * KB, &tm_kv, h * 64, off, kvh, page, 1, &v_full[s]);
          ++v_issued;
        }
      }
      if (gave_up) {
        // let copies already in flight land before the CTA (and its shared memory) goes away
        const unsigned long long start = global_ns();
        while (!mbar_try(&q_full, 0) && global_ns() - start < 100000000ull) {}
        for (int j = k_issued > 2 ? k_issued - 2 : 0; j < k_issued; ++j) {
          const unsigned long long t0 = global_ns();
          while (!mbar_try(&k_full[j & 1], ((unsigned)j >> 1) & 1u) && global_ns() - t0 < 100000000ull) {}
        }
        for (int j = v_issued > 2 ? v_issued - 2 : 0; j < v_issued; ++j) {
          const unsigned long long t0 = global_ns();
          while (!mbar_try(&v_full[j & 1], ((unsigned)j >> 1) & 1u) && global_ns() - t0 < 100000000ull) {}
        }
      }
    }
    // P is 0 at keys past the segment's end, but 0 * V must stay 0 even if an earlier
    // request left a NaN or an infinity in the page: once the last V tile has landed
    // this warp zeroes those rows (128 bytes per 64 head dims), then lets the O product go.
    __syncwarp();
    if (stale_from < AK && !gave_up) {
      const int j = ntiles - 1;
      bool ok = mbar_wait(&v_full[j & 1], ((unsigned)j >> 1) & 1u, &gave_up);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok) {
        for (int idx = lane; idx < NB * AK; idx += 32) {
          const int rr = idx % AK, hb = idx / AK;
          if (rr >= stale_from) {
            uint4* row = reinterpret_cast<uint4*>(sVr + (j & 1) * K_BYTES + hb * KB + rr * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) row[c] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&v_clean);
      } else if (lane == 0) {
        atomicCAS(a.status, 0, FT_ST_PREFILL_CLEANER);
        gave_up = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptors: D f32, A/B bf16, M = 128; S: N = 64, both K-major;
      // O: N = D, B (= V) MN-major
      const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AK >> 3) << 17) |
                               ((unsigned)(AQ >> 4) << 24);
      const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) |
                               ((unsigned)(AQ >> 4) << 24);
      bool ok = mbar_wait(&q_full, 0, &gave_up);
      if (!ok) { atomicCAS(a.status, 0, FT_ST_PREFILL_MMA_Q); gave_up = 1; }
      const unsigned sQa = smem_u32(sQ);
      // S product of tile j into S buffer j & 1; frees the K stage when done
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], ((unsigned)j >> 1) & 1u, &gave_up)) {
          atomicCAS(a.status, 0, FT_ST_PREFILL_MMA_K);
          gave_up = 1;
          return false;
        }
        tc_fence_after();
        const unsigned sK = smem_u32(sKr + s * K_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma(tmem_s + (unsigned)(s * AK), sw128_desc(sQa + (kk >> 2) * QB + (kk & 3) * 32),
                 sw128_desc(sK + (kk >> 2) * KB + (kk & 3) * 32), idesc_s, kk > 0);
        tc_commit(&s_full[s]);
        tc_commit(&k_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        // the next tile's S goes first: it runs under this tile's softmax.  Its buffer
        // held P of tile j-1, read by an O product issued before it (MMAs run in order)
        if (j + 1 < ntiles && !issue_s(j + 1)) break;
        if (!mbar_wait(&p_full[s], ((unsigned)j >> 1) & 1u, &gave_up) ||
            !mbar_wait(&v_full[s], ((unsigned)j >> 1) & 1u, &gave_up) ||
            (j == ntiles - 1 && stale_from < AK && !mbar_wait(&v_clean, 0, &gave_up))) {
          atomicCAS(a.status, 0, FT_ST_PREFILL_MMA_PV);
          gave_up = 1;
          break;
        }
        tc_fence_after();
        const unsigned sV = smem_u32(sVr + s * K_BYTES);
#pragma unroll
        for (int kk = 0; kk < AK / 16; ++kk)
          tc_mma_ts(tmem_o, tmem_s + (unsigned)(s * AK + kk * 8), sw128_mn_desc(sV + kk * 16 * 128, KB, 1024),
                    idesc_o, (j | kk) != 0);
        tc_commit(&v_empty[s]);
        tc_commit(&pv_done);
      }
    }
  } else {
    // softmax: TMEM lane = query row; this warp may touch lanes 32*(warp%4) .. +31
    const int lane_base = (warp & 3) * 32;
    const int r = lane_base + lane;
    const int my_tok = r % TOK, my_head = head + r / TOK;
    const int my_pos = pos_first + my_tok;
    const unsigned lane_bits = (unsigned)lane_base << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const unsigned tmem_sj = tmem_s + (unsigned)((j & 1) * AK) + lane_bits;
      ok = mbar_wait(&s_full[j & 1], ((unsigned)j >> 1) & 1u, &gave_up);
      if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_PREFILL_SOFTMAX_S); gave_up = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      unsigned lo[32], hi[32];
      tc_ld32(tmem_sj, lo);
      tc_ld32(tmem_sj + 32, hi);
      tc_ld_wait();
      const int key0 = j * AK;
      if (key0 + AK - 1 > pos_first) {
        // a tile on the diagonal: keys after the row's own position do not count
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (key0 + c > my_pos) lo[c] = 0xff800000u;
          if (key0 + 32 + c > my_pos) hi[c] = 0xff800000u;
        }
      }
      // four independent chains each for the max and (below) the sum: two warps per
      // scheduler cannot hide one long dependent chain
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; ++c)
        mx4[c & 3] = fmaxf(mx4[c & 3], fmaxf(__uint_as_float(lo[c]), __uint_as_float(hi[c])));
      const float raw = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The running max only moves when it would grow by more than 2^8: below
      // that exp2(s - max) stays far inside float32 and bfloat16 range, and the
      // round trip of O through registers is saved.  The softmax is the same
      // function of the scores whichever offset is subtracted.
      const float cand = raw * a.scale_log2;
      const float m_new = cand > m + 8.f ? cand : m;
      if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
        // O must be at rest: the previous tile's O product done (the one before it
        // is, since this tile's S product was issued after it), this tile's not issued
        ok = mbar_wait(&pv_done, (unsigned)(j - 1) & 1u, &gave_up);
        if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_PREFILL_SOFTMAX_PV); gave_up = 1; }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tc_fence_after();
        const float alpha = fast_exp2(m - m_new);
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          unsigned o[32];
          tc_ld32(tmem_o + lane_bits + c0, o);
          tc_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tc_st32(tmem_o + lane_bits + c0, o);
        }
        tc_st_wait();
        l *= alpha;
      }
      m = m_new;
      // P = exp2(s * scale - max), summed in float32, rounded to bfloat16 and written
      // over S: column c of the buffer holds keys 2c and 2c+1
      const float neg_m = -m_new;
      // packed pairs: one fma.rn.f32x2 / add.f32x2 does two elements
      const float2 sc2 = make_float2(a.scale_log2, a.scale_log2), nm2 = make_float2(neg_m, neg_m);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      unsigned pk[32];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(lo[2 * c]), __uint_as_float(lo[2 * c + 1])), sc2, nm2);
        const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(hi[2 * c]), __uint_as_float(hi[2 * c + 1])), sc2, nm2);
        const float2 p01 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
        const float2 p23 = make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
        sum2[c & 3] = __fadd2_rn(sum2[c & 3], __fadd2_rn(p01, p23));
        pk[c] = pack_bf16(p01.x, p01.y);
        pk[16 + c] = pack_bf16(p23.x, p23.y);
      }
      const float2 s01 = __fadd2_rn(__fadd2_rn(sum2[0], sum2[1]), __fadd2_rn(sum2[2], sum2[3]));
      const float sum = s01.x + s01.y;
      tc_st32(tmem_sj, pk);
      tc_st_wait();
      l += sum;
      if (j == ntiles - 1 && j > 0) {
        // A parity wait tells the phase it asks for from the one two earlier only
        // while the waiter is at most one phase behind.  The wait after the loop asks
        // for the O product of this last tile; this warp may have run ahead of its
        // siblings (S of this tile was issued before the O product of tile j-1, which
        // waits for all four warps and for V), so that product may not be done and the
        // barrier would still be in phase j-1: the final wait would then be answered
        // by phase j-2 and O read two products early.  Waiting here for product j-1,
        // BEFORE this warp's arrival lets product j go, pins the phase.
        ok = mbar_wait(&pv_done, (unsigned)(j - 1) & 1u, &gave_up);
        if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_PREFILL_SOFTMAX_PV); gave_up = 1; }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
    }
    if (ok) {
      ok = mbar_wait(&pv_done, (unsigned)(ntiles - 1) & 1u, &gave_up);
      if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_PREFILL_SOFTMAX_LAST); gave_up = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + ((size_t)(tok0 + my_tok) * a.nq + my_head) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        unsigned o[32];
        tc_ld32(tmem_o + lane_bits + c0, o);
        tc_ld_wait();
        if (my_tok < rows) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + c) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int D, int HPC>
int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mq2, const CUtensorMap& mkv,
                      const PrefillTcArgs& a, int tiles, cudaStream_t stream) {
  constexpr int NB = D / 64;
  constexpr int K_BYTES = NB * AK * 128;
  const size_t smem = (size_t)NB * AQ * 128 + 4 * K_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D, HPC>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(tiles, a.nq / HPC);
  attn_prefill_tc_kernel<D, HPC><<<grid, 192, smem, stream>>>(mq, mq2, mkv, a);
  return FT_OK;
}

}  // namespace ft

using namespace ft;

extern "C" {

// Tensor map over the bfloat16 query rows [rows, cols] (row stride in elements):
// boxes of `box_rows` (128 or 64) rows by 64 columns in the 128-byte swizzle.
// `out` receives 128 bytes.
int ft_attn_tc_q_map(void* out, const void* base, long long rows, long long cols, long long row_stride,
                     int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -201;
  if ((cols & 7) || (row_stride & 7) || ((uintptr_t)base & 15) || (box_rows != AQ && box_rows != AQ / 2))
    return FT_ERR_SHAPE;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return -202;
  memcpy(out, &map, sizeof(map));
  return FT_OK;
}

// Tensor map over one layer's pages, bfloat16 [2, pages, nkv, P, d] with the
// given strides (elements) of the three outer dimensions: boxes of 64 keys by
// 64 head dims of one page, one head, K or V.
int ft_attn_tc_kv_map(void* out, const void* base, long long pages, long long nkv, long long P, long long d,
                      long long head_stride, long long page_stride, long long kv_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -201;
  if ((d & 63) || P < AK || (head_stride & 7) || (page_stride & 7) || (kv_stride & 7) || ((uintptr_t)base & 15))
    return FT_ERR_SHAPE;
  CUtensorMap map;
  cuuint64_t dims[5] = {(cuuint64_t)d, (cuuint64_t)P, (cuuint64_t)nkv, (cuuint64_t)pages, 2};
  cuuint64_t strides[4] = {(cuuint64_t)d * 2, (cuuint64_t)head_stride * 2, (cuuint64_t)page_stride * 2,
                           (cuuint64_t)kv_stride * 2};
  cuuint32_t box[5] = {64, AK, 1, 1, 1};
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  CUresult rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, (void*)base, dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return -202;
  memcpy(out, &map, sizeof(map));
  return FT_OK;
}

// bfloat16; head_dim 64 or 128; page size a multiple of 64; no window.
// tile_seg / tile_q0 list the query tiles (64 tokens) of the segments to
// process.  With an even number of query heads per KV head a CTA takes one tile
// and two heads (`map_q2`: boxes of 64 rows); otherwise an even tile with its
// successor and one head (`map_q`: boxes of 128 rows).
int ft_attn_prefill_tc(const void* map_q, const void* map_q2, const void* map_kv, void* out, const int* tile_seg,
                       const int* tile_q0, const int* seg_q_start, const int* seg_pos0,
                       const int* block_table, int* status, int nq, int nkv, int d, int P,
                       int table_width, int tiles, float scale, cudaStream_t stream) {
  if (tiles <= 0) return FT_OK;
  if (nkv <= 0 || nq % nkv || P % AK) return FT_ERR_SHAPE;
  CUtensorMap mq, mq2, mkv;
  memcpy(&mq, map_q, sizeof(mq));
  memcpy(&mq2, map_q2, sizeof(mq2));
  memcpy(&mkv, map_kv, sizeof(mkv));
  const bool pair = ((nq / nkv) % 2) == 0;
  PrefillTcArgs a{(__nv_bfloat16*)out, tile_seg, tile_q0, seg_q_start, seg_pos0, block_table, status,
                  nq, nkv, P, table_width, scale * 1.4426950408889634f};
  int rc;
  switch (d) {
    case 64:
      rc = pair ? launch_prefill_tc<64, 2>(mq, mq2, mkv, a, tiles, stream)
                : launch_prefill_tc<64, 1>(mq, mq2, mkv, a, tiles, stream);
      break;
    case 128:
      rc = pair ? launch_prefill_tc<128, 2>(mq, mq2, mkv, a, tiles, stream)
                : launch_prefill_tc<128, 1>(mq, mq2, mkv, a, tiles, stream);
      break;
    default: return FT_ERR_SHAPE;
  }
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
