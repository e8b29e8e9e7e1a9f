// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands staged in shared memory by TMA.
//
// For every expert e that has rows (sorted routes off[e]..off[e+1]), every tile
// of its tokens and every tile of its weight rows one accumulator in TMEM, in one
// of two forms:
//   weight-major   D[128 weight rows, N tokens] = W_e tile * X^T: the WEIGHTS are the M
//                  operand of the MMA (always a full 128-row tile), the TOKENS the N
//                  operand (N = 16..128, as many as the tile holds), so an expert with
//                  few tokens wastes little of the tensor core
//   token-major    D[128 tokens, 256 weight rows] = X tile * W_e tile^T: a TMEM lane is a
//                  token, the columns are consecutive output features
// Both operands are K-major, so neither form needs a transpose.  Accumulation is
// float32 in TMEM.
//
//   warp 0     TMA producer: per 64-wide k-block two weight boxes of 128 rows and one
//              token box into a ring of stages, completion on the stage's "full"
//              mbarrier
//   warp 1     allocates TMEM; one thread issues tcgen05.mma (K = 16) four (eight) per
//              k-block, then tcgen05.commit to the stage's "empty" mbarrier, and after
//              the last k-block to the "accumulator" one
//   warps 2-5  epilogue: tcgen05.ld the accumulator, GLU: act(gate)*up; down: * route
//              weight in float32; round; store into [token, feature] rows
// The kernel is persistent (one CTA per SM) and the accumulator has two TMEM
// buffers, so a tile's epilogue runs while the next tile's k-blocks stream in.
//
// Every mbarrier wait is bounded (about two seconds): on expiry the CTA writes
// a code into `status`, stops issuing work, frees its TMEM and returns.
//
// Reference counterpart: python/freetoken/kernel/triton/fused_moe.py:156-302
// (tl.dot grouped GEMM over block-padded sorted tokens),
// python/freetoken/kernel/triton/activation.py:96-107 (activation as its own
// kernel), weight multiply at fused_moe.py:292-296.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "tcgen05.cuh"

namespace ft {

constexpr int TC_BM = 128;         // rows of the M operand (UMMA M)
constexpr int TC_BK = 64;          // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_MAXN = 128;       // most tokens per tile
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;     // 16 KB: a box of 128 rows

struct TcArgs {
  void* C;
  const int4* tile_info;      // [tiles_bound]: {expert (-1 past the end), first sorted row, rows the MMA
                              // covers (rounded up to 16), end of the expert's rows} of each token tile
  const int* c_rows;          // sorted row -> output row, or nullptr
  const float* row_scale;     // by output row, or nullptr
  int* status;                // 0 = fine; otherwise the first failure code
  long long ldc;
  int n_out;                  // output features (weight rows; with GLU: rows of each half)
  int K, ntok, tiles_y;
  int act;
  float act_alpha, act_limit;
};

__device__ __forceinline__ float tc_glu(float g, float u, int act, float alpha, float limit) {
  if (act == 0) return (g / (1.f + __expf(-g))) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return (g / (1.f + __expf(-alpha * g))) * (u + 1.f);
}

// Rows of one token tile of a group with `r` rows when tiles hold at most `ntok`: the
// group's rows are dealt out evenly over the fewest tiles that hold them (in steps of
// 16, the MMA's N granularity).  An expert with 140 rows gets two tiles of 80 rather
// than one of 128 and one of 12 - in the weight-major form the short tile would stream
// the whole weight tile for a sliver of work.
__host__ __device__ __forceinline__ int tc_tile_rows(int r, int ntok) {
  const int nt = (r + ntok - 1) / ntok;
  if (nt <= 1) return ntok;
  const int sz = (((r + nt - 1) / nt) + 15) & ~15;
  return sz < ntok ? sz : ntok;
}

// Kernel variants.
//   TC_GLU2   gate_up + GLU, weight-major: 128 output features per tile as TWO accumulators
//             (128 gate rows, 128 up rows) of up to 128 tokens.  For few rows per expert,
//             where the step is bound by streaming each expert's weights once and a tile
//             should cost no more products than it holds tokens.
//   TC_GLUT   gate_up + GLU, token-major: 128 gate rows and the 128 up rows of the same
//             features lie one after the other in shared memory as ONE N operand of 256,
//             so the accumulator's columns c and c + 128 are gate and up of feature c in
//             the same lane.  For busy experts (the M tile is always 128 rows).
//   TC_TOK    no GLU (the down projection), token-major: 256 weight rows (two boxes of
//             128) are the N operand, 256 output features per tile.
// In the token-major forms a thread of the epilogue owns a token and writes 16 consecutive
// features with two 16-byte stores.  Weight-major forms of the down projection (a thread
// owns a feature and writes one 2-byte value per token; tiles of up to 128 or 256 tokens)
// were the first ones built: at 256 rows per expert their 2-byte stores, not the products,
// set the pace (measured with per-role cycle counters: the epilogue warps busy 90 % of the
// kernel's time, the MMA warp waiting for a free accumulator 28 % of it; without the
// stores the kernel ran 1.67 times as fast).  Token-major is level with them up to 192
// rows per expert and 10-30 % faster beyond (256 experts of real width, 8,192 tokens:
// 734 against 812 us; 64 experts with 512 rows each: 346 against 485 us), so they went.
// Measured against TC_GLU2, TC_GLUT takes 905 against 919 us at 128 rows per expert, 1,115
// against 1,191 at 192, 1,343 against 1,480 at 256, 2,274 against 2,683 at 512; at 64 rows
// 767 against 758.
//
// Also built, measured and dropped:
//  * gate and up rows side by side in ONE weight-major accumulator of up to 256 tokens
//    (642 instead of 392 us at 256 rows per expert: pairing TMEM lane f with lane f + 64
//    through shared memory does not hide under the main loop);
//  * an expert's short last tile run weight-major inside the token-major kernel (N as
//    narrow as its rows): slower, a tile costs its bytes, not its products;
//  * CTA pairs (`cta_group::2`, a cluster of two CTAs on one tile of 256 tokens by 256
//    weight rows, each CTA loading 128 of both, 32 instead of 48 KB per k-block, the
//    even CTA issuing MMAs of M = 256; bit-equal results): 765 against 734 us (down)
//    and 1,520 against 1,343 us (gate_up) at 256 rows per expert, level at 512, 9 % ahead
//    only at 2,500 rows per expert (down): tiles of 256 tokens pad more than they save.
enum { TC_GLU2 = 0, TC_GLUT = 1, TC_TOK = 2 };

// Persistent: one CTA per SM walks the tiles t = blockIdx.x, + gridDim.x, ...
// of the (token tile, weight tile) space, weight tile fastest, so CTAs that run
// side by side share an expert.  The TMA ring never drains between tiles and the
// accumulator is double-buffered in TMEM, so the epilogue of one tile runs under
// the main loop of the next.  The token rows come through one of two tensor maps
// with boxes of 64 or 128 rows: the smaller when it holds the tile.
template <int MODE>
__global__ void __launch_bounds__(192) moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                          const __grid_constant__ CUtensorMap tm_x0,
                                                          const __grid_constant__ CUtensorMap tm_x1,
                                                          TcArgs a) {
  constexpr bool GLUT = MODE == TC_GLUT, TOK = MODE == TC_TOK;   // else TC_GLU2
  constexpr bool TMAJ = GLUT || TOK;                  // tokens are the M operand
  // a stage: two boxes of 128 weight rows (gate and up rows of the same features, or 256
  // consecutive rows) and up to 128 token rows of one 64-wide k-block: 40 or 48 KB
  constexpr int STAGES = 4;
  constexpr int STAGE_BYTES = 3 * TC_A_BYTES;
  constexpr int FEAT = TOK ? 2 * TC_BM : TC_BM;       // output features per tile
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  __shared__ volatile int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntok = a.ntok;
  const int acc_cols = TMAJ ? 2 * TC_BM : 2 * ntok;   // columns of one accumulator buffer
  const unsigned tmem_cols = 2 * acc_cols <= 32 ? 32u : (2 * acc_cols <= 64 ? 64u :
                             (2 * acc_cols <= 128 ? 128u : (2 * acc_cols <= 256 ? 256u : 512u)));
  if (threadIdx.x == 0) {
    gave_up = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  const int kblocks = (a.K + TC_BK - 1) / TC_BK;
  const int wtiles = (a.n_out + FEAT - 1) / FEAT;
  const int total = a.tiles_y * wtiles;
  // A role reads the entry of its NEXT tile while it works on the current one: under load
  // a load from global memory takes microseconds, and a tile's first copy or product must
  // not wait for it.  Tiles are in order, so nothing follows an empty entry.
  auto tile_at = [&](int t) { return t < total ? __ldg(&a.tile_info[t / wtiles]) : make_int4(-1, 0, 0, 0); };

  if (warp == 0) {
    if (lane == 0) {
      long long issued = 0;           // k-blocks issued so far, over all tiles
      bool ok = true;
      int4 cur = tile_at(blockIdx.x);
      for (int t = blockIdx.x; t < total && ok && cur.x >= 0; t += gridDim.x) {
        const int4 nxt = tile_at(t + gridDim.x);
        const int n0 = (t % wtiles) * FEAT;
        const int e = cur.x, row0 = cur.y;
        // the second box of weight rows: the up rows of the same features, or the next 128 rows
        const int n1 = TOK ? n0 + TC_BM : a.n_out + n0;
        const bool small = cur.z <= 64;
        const CUtensorMap* tm_x = small ? &tm_x0 : &tm_x1;
        const unsigned tx = 2 * TC_A_BYTES + (small ? 64u : 128u) * TC_BK * 2;
        for (int kb = 0; kb < kblocks; ++kb, ++issued) {
          const int s = (int)(issued % STAGES);
          const unsigned ph = (unsigned)(issued / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_MOE_PRODUCER);
            gave_up = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], tx);
          // a k-block past K is all zero fill and still counts its bytes
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          const int k = kb * TC_BK;
          tma_load_3d(st, &tm_w, k, n0, e, &full_bar[s]);
          tma_load_3d(st + TC_A_BYTES, &tm_w, k, n1, e, &full_bar[s]);
          tma_load_2d(st + 2 * TC_A_BYTES, tm_x, k, row0, &full_bar[s]);
        }
        cur = nxt;
      }
      if (gave_up) {
        // let copies already in flight land before the CTA (and its shared memory) goes away
        for (long long kb = issued > STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
          const unsigned long long start = global_ns();
          while (!mbar_try(&full_bar[kb % STAGES], (unsigned)(kb / STAGES) & 1u) &&
                 global_ns() - start < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      long long done = 0;             // k-blocks consumed so far
      int local = 0;                  // tiles this CTA has started
      bool ok = true;
      int4 cur = tile_at(blockIdx.x);
      for (int t = blockIdx.x; t < total && ok && cur.x >= 0; t += gridDim.x) {
        const int4 nxt = tile_at(t + gridDim.x);
        // instruction descriptor: D f32, A/B bf16, both K-major, M = 128; weight-major: N =
        // the rows this tile really has, rounded up to 16 (a tile costs what it holds);
        // token-major: N = 256 weight rows
        const int n_tile = cur.z;
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((unsigned)((TMAJ ? 2 * TC_BM : n_tile) >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((unsigned)(local >> 1) & 1u) ^ 1u, &gave_up)) {
          atomicCAS(a.status, 0, FT_ST_MOE_MMA_ACC);
          gave_up = 1;
          break;
        }
        tc_fence_after();
        const unsigned tmem_d = tmem_base + (unsigned)(b * acc_cols);
        for (int kb = 0; kb < kblocks; ++kb, ++done) {
          const int s = (int)(done % STAGES);
          const unsigned ph = (unsigned)(done / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_MOE_MMA_STAGE);
            gave_up = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const unsigned st = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const unsigned sx = st + 2 * TC_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk) {
            const unsigned acc = (kb | kk) != 0;
            const unsigned long long xdesc = sw128_desc(sx + kk * 32);
            if constexpr (TMAJ) {          // A: the token rows; B: the two boxes of weight rows, 256 in all
              tc_mma(tmem_d, xdesc, sw128_desc(st + kk * 32), idesc, acc);
            } else {                       // A: gate rows, then up rows; B: the token rows
              tc_mma(tmem_d, sw128_desc(st + kk * 32), xdesc, idesc, acc);
              tc_mma(tmem_d + ntok, sw128_desc(st + TC_A_BYTES + kk * 32), xdesc, idesc, acc);
            }
          }
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&acc_full[b]);
        ++local;
        cur = nxt;
      }
    }
  } else {
    // epilogue: this warp may touch TMEM lanes 32*(warp%4) .. +31
    const int lane_base = (warp & 3) * 32;
    __nv_bfloat16* C = (__nv_bfloat16*)a.C;
    int local = 0;
    int4 cur = tile_at(blockIdx.x);
    for (int t = blockIdx.x; t < total && cur.x >= 0; t += gridDim.x) {
      const int4 nxt = tile_at(t + gridDim.x);
      const int row0 = cur.y, row_end = cur.w;
      const int b = local & 1;
      const int n_tile = cur.z;
      const int n0 = (t % wtiles) * FEAT;
      // token-major: this thread's token, its output row and route weight, fetched before
      // the accumulator is waited for
      const int row = row0 + lane_base + lane;
      const bool valid = TMAJ && lane_base + lane < n_tile && row < row_end;
      const int crow = valid ? (a.c_rows ? a.c_rows[row] : row) : 0;
      const float scale = valid && a.row_scale ? a.row_scale[crow] : 1.f;
      bool ok = mbar_wait(&acc_full[b], (unsigned)(local >> 1) & 1u, &gave_up);
      if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_MOE_EPILOGUE); gave_up = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const unsigned tmem_d = tmem_base + (unsigned)(b * acc_cols) + ((unsigned)lane_base << 16);
      if constexpr (TMAJ) {
        // TMEM lane = token row of the tile.  GLU: columns c and c + 128 are gate and up of
        // feature n0 + c; otherwise column c is feature n0 + c, 256 of them
        __nv_bfloat16* dst = C + (size_t)crow * a.ldc + n0;
        const bool vec = (a.ldc & 7) == 0 && ((uintptr_t)C & 15) == 0;
        for (int c0 = 0; c0 < FEAT && n0 + c0 < a.n_out; c0 += 16) {
          unsigned g[16], u[16];
          tc_ld16(tmem_d + (unsigned)c0, g);
          if (GLUT) tc_ld16(tmem_d + (unsigned)(TC_BM + c0), u);
          tc_ld_wait();
          if (!valid) continue;
          unsigned packed[8];
#pragma unroll
          for (int c = 0; c < 16; c += 2) {
            float v0, v1;
            if (GLUT) {
              v0 = scale * tc_glu(__uint_as_float(g[c]), __uint_as_float(u[c]), a.act, a.act_alpha, a.act_limit);
              v1 = scale * tc_glu(__uint_as_float(g[c + 1]), __uint_as_float(u[c + 1]), a.act, a.act_alpha, a.act_limit);
            } else {
              v0 = __uint_as_float(g[c]) * scale;
              v1 = __uint_as_float(g[c + 1]) * scale;
            }
            const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            packed[c >> 1] = *reinterpret_cast<const unsigned*>(&h);
          }
          if (vec && n0 + c0 + 16 <= a.n_out) {
            *reinterpret_cast<uint4*>(dst + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (n0 + c0 + c < a.n_out) {
                const unsigned w = packed[c >> 1];
                const unsigned short bits = (c & 1) ? (unsigned short)(w >> 16) : (unsigned short)(w & 0xffffu);
                dst[c0 + c] = __ushort_as_bfloat16(bits);
              }
          }
        }
      } else {
        // weight-major GLU: TMEM lane = feature n; column c of the two accumulators = gate
        // and up of the tile's token c, whose output row is its sorted row
        const int n = n0 + lane_base + lane;
        for (int c0 = 0; c0 < n_tile; c0 += 16) {
          unsigned g[16], u[16];
          tc_ld16(tmem_d + (unsigned)c0, g);
          tc_ld16(tmem_d + (unsigned)(c0 + ntok), u);
          tc_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int r = row0 + c0 + c;
            if (r < row_end && n < a.n_out) {
              const int cr = a.c_rows ? a.c_rows[r] : r;
              float v = tc_glu(__uint_as_float(g[c]), __uint_as_float(u[c]), a.act, a.act_alpha, a.act_limit);
              if (a.row_scale) v *= a.row_scale[cr];
              C[(size_t)cr * a.ldc + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
      ++local;
      cur = nxt;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// tile_info[y] = {expert, first sorted row, rows the MMA covers (rounded up to 16), end of
// the expert's rows} for every (busy expert, tile of ntok rows), in expert order; entries
// past the last tile get expert -1.  One block.
__global__ void moe_tile_map_kernel(const int* __restrict__ group_offsets, const int* __restrict__ active,
                                    int4* __restrict__ tile_info, int G, int ntok, int bound) {
  __shared__ int scan[1024];
  __shared__ int carry;
  const int busy = active[G];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < busy; base += blockDim.x) {
    const int j = base + threadIdx.x;
    int e = -1, begin = 0, end = 0, nt = 0, sz = ntok;
    if (j < busy) {
      e = active[j];
      begin = group_offsets[e];
      end = group_offsets[e + 1];
      const int r = end - begin;
      nt = (r + ntok - 1) / ntok;
      sz = tc_tile_rows(r, ntok);        // the group's rows dealt out evenly over its tiles
    }
    scan[threadIdx.x] = nt;
    __syncthreads();
    // inclusive scan (Hillis-Steele) over the block
    for (int o = 1; o < (int)blockDim.x; o <<= 1) {
      const int v = threadIdx.x >= (unsigned)o ? scan[threadIdx.x - o] : 0;
      __syncthreads();
      scan[threadIdx.x] += v;
      __syncthreads();
    }
    const int first = carry + scan[threadIdx.x] - nt;
    for (int i = 0; i < nt && first + i < bound; ++i) {
      const int row0 = begin + i * sz;
      tile_info[first + i] = make_int4(e, row0, min(sz, (end - row0 + 15) & ~15), end);
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry += scan[threadIdx.x];
    __syncthreads();
  }
  for (int i = carry + threadIdx.x; i < bound; i += blockDim.x) tile_info[i] = make_int4(-1, 0, 0, 0);
}

// Exercises the bounded wait itself: thread 0 waits (at most `limit_ns`) on an
// mbarrier that thread 1 arrives at only when `arrive` is set.  When the wait
// runs out the thread records its code in the status word, as every role of the
// kernels above does, and the kernel returns normally.
__global__ void wait_selftest_kernel(int* status, unsigned long long limit_ns, int arrive) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ volatile int gave_up;
  if (threadIdx.x == 0) {
    gave_up = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 1 && arrive) mbar_arrive(&bar);
  if (threadIdx.x == 0 && !mbar_wait(&bar, 0, &gave_up, limit_ns)) {
    atomicCAS(status, 0, FT_ST_SELFTEST_WAIT);
    gave_up = 1;
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

template <int MODE>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap* mx, const TcArgs& a, dim3 grid, size_t smem,
                     cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  moe_gemm_tc_kernel<MODE><<<grid, 192, smem, stream>>>(mw, mx[0], mx[1], a);
  return FT_OK;
}

}  // namespace ft

using namespace ft;

extern "C" {

// Tensor map over bfloat16 rows with boxes of [box_rows, 64] in the 128-byte swizzle:
// 3-D [groups, rows, K] for the expert weights (`groups` >= 1: the kernel addresses them
// with three coordinates, one expert or many), 2-D [rows, K] for the token rows
// (`groups` = 0).  The rank must be the rank of the load that uses the map: a 3-D load
// through a 2-D map is an illegal instruction.  `out` receives 128 bytes.
int ft_tc_make_map(void* out, const void* base, long long groups, long long rows, long long K,
                   long long row_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -201;
  if ((K & 7) || (row_stride & 7) || ((uintptr_t)base & 15) || box_rows < 1 || box_rows > 256) return FT_ERR_SHAPE;
  CUtensorMap map;
  CUresult rc;
  if (groups >= 1) {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)groups};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)rows * (cuuint64_t)row_stride * 2};
    cuuint32_t box[3] = {TC_BK, (cuuint32_t)box_rows, 1};
    cuuint32_t es[3] = {1, 1, 1};
    rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)base, dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1, 1};
    rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (rc != CUDA_SUCCESS) return -202;
  memcpy(out, &map, sizeof(map));
  return FT_OK;
}

// One block whose first thread waits up to `limit_ns` nanoseconds (at most a
// second) on a barrier that is arrived at only if `arrive` is non-zero; a wait
// that runs out leaves FT_ST_SELFTEST_WAIT in `status`.
int ft_wait_selftest(int* status, long long limit_ns, int arrive, cudaStream_t stream) {
  if (!status || limit_ns < 0 || limit_ns > 1000000000ll) return FT_ERR_SHAPE;
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, (unsigned long long)limit_ns, arrive);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// C rows (bfloat16) for the sorted rows of every busy expert.  map_w: 3-D map of
// the expert weights (box 128 rows); map_x: 2-D map of the sorted token rows
// (box `ntok` rows).  rows_bound: most sorted rows there can be.
// How many (expert, token tile) entries a tile map for `rows_bound` sorted rows needs.
int ft_tc_tiles_bound(int rows_bound, int G, int ntok) {
  return (rows_bound + ntok - 1) / ntok + (G < rows_bound ? G : rows_bound);
}

int ft_moe_tile_map(const int* group_offsets, const int* active, void* tile_info,
                    int rows_bound, int G, int ntok, cudaStream_t stream) {
  if (ntok < 1 || G <= 0 || ((uintptr_t)tile_info & 15)) return FT_ERR_SHAPE;
  const int bound = ft_tc_tiles_bound(rows_bound, G, ntok);
  moe_tile_map_kernel<<<1, 256, 0, stream>>>(group_offsets, active, (int4*)tile_info, G, ntok, bound);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// `map_w`: the 3-D map of the expert weights with boxes of 128 rows.  `maps_x`: two 2-D
// maps of the sorted token rows, 128 bytes each, with boxes of 64 and 128 rows.
// `ntok`: most rows of a token tile, as the tile list was made (a multiple of 16, at most
// 128); `G`: the number of experts.  `form`: 0 gate_up + GLU weight-major (TC_GLU2), 1 gate_up
// + GLU token-major (TC_GLUT), 2 no GLU, token-major (TC_TOK).
int ft_moe_gemm_tc(const void* map_w, const void* maps_x, void* C, long long ldc, const void* tile_info,
                   const int* c_rows, const float* row_scale, int* status, int rows_bound, int n_out,
                   int K, int G, int ntok, int form, int act, float act_alpha, float act_limit,
                   cudaStream_t stream) {
  if (rows_bound <= 0 || n_out <= 0) return FT_OK;
  if (ntok < 16 || ntok > TC_MAXN || (ntok & 15) || (K & 7) || G <= 0 || form < 0 || form > 2) return FT_ERR_SHAPE;
  CUtensorMap mw, mx[2];
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(mx, maps_x, sizeof(mx));
  const int tiles_y = ft_tc_tiles_bound(rows_bound, G, ntok);
  TcArgs a{C, (const int4*)tile_info, c_rows, row_scale, status, ldc, n_out, K, ntok, tiles_y, act, act_alpha,
           act_limit};
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int feat = form == TC_TOK ? 2 * TC_BM : TC_BM;
  const int total = tiles_y * ((n_out + feat - 1) / feat);
  dim3 grid(total < sms ? total : sms);
  const size_t smem = 4 * 3 * TC_A_BYTES + 1024;
  int rc;
  if (form == TC_TOK) rc = launch_tc<TC_TOK>(mw, mx, a, grid, smem, stream);
  else if (form == TC_GLUT) rc = launch_tc<TC_GLUT>(mw, mx, a, grid, smem, stream);
  else rc = launch_tc<TC_GLU2>(mw, mx, a, grid, smem, stream);
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
