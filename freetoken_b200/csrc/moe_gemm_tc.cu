// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands staged in shared memory by TMA.
//
// For every expert e that has rows (sorted routes off[e]..off[e+1]) and every
// tile of 128 weight rows:   D[128 weight rows, N tokens] = W_e tile * X^T
// The WEIGHTS are the M operand of the MMA (always a full 128-row tile, whatever
// the load of the expert), the expert's TOKENS are the N operand (N = 16..128
// per tile), both K-major, so neither needs a transpose and an expert with few
// tokens wastes little of the tensor core.  Accumulation is float32 in TMEM.
//
//   warp 0     TMA producer: per 64-wide k-block one weight box (two with GLU:
//              gate rows and up rows) and one token box into a ring of stages,
//              completion on the stage's "full" mbarrier
//   warp 1     allocates TMEM; one thread issues tcgen05.mma (M=128, N, K=16)
//              four per k-block, then tcgen05.commit to the stage's "empty"
//              mbarrier, and after the last k-block to the "accumulator" one
//   warps 2-5  epilogue: tcgen05.ld the accumulator (a thread owns one weight
//              row = one TMEM lane), GLU: act(gate)*up; down: * route weight in
//              float32; round; store transposed into [token, feature] rows
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

constexpr int TC_BM = 128;         // weight rows per tile (UMMA M)
constexpr int TC_BK = 64;          // k-block: 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_MAXN = 128;       // most tokens per tile (UMMA N); 256 in the wide build
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;     // 16 KB

struct TcArgs {
  void* C;
  const int* group_offsets;   // [G+1]
  const int* active;          // [G+1]: experts with rows, then their number
  const int4* tile_info;      // [tiles_bound]: {expert (-1 past the end), first sorted row, rows the MMA
                              // covers (rounded up to 16), end of the expert's rows} of each token tile
  const int* c_rows;          // sorted row -> output row, or nullptr
  const float* row_scale;     // by output row, or nullptr
  int* status;                // 0 = fine; otherwise the first failure code
  long long ldc;
  int n_out;                  // output features (weight rows; with GLU: rows of each half)
  int K, G, ntok, tiles_y;
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
// 16, the MMA's N granularity).  An expert with 280 rows and 256-row tiles gets two
// tiles of 144 rather than one of 256 and one of 24 - the short tile would stream the
// whole weight tile for a sliver of work.
__host__ __device__ __forceinline__ int tc_tile_rows(int r, int ntok) {
  const int nt = (r + ntok - 1) / ntok;
  if (nt <= 1) return ntok;
  const int sz = (((r + nt - 1) / nt) + 15) & ~15;
  return sz < ntok ? sz : ntok;
}

// Kernel variants.
//   TC_GLU2   gate_up + GLU, 128 output features per tile as TWO accumulators (128 gate
//             rows, 128 up rows), up to 128 tokens: few rows per expert, where the step
//             is bound by streaming each expert's weights once
//   TC_PLAIN  no GLU, 128 weight rows x up to 128 tokens, two k-blocks per stage
//   TC_WIDE   no GLU, 128 weight rows x up to 256 tokens
//   TC_GLUT   gate_up + GLU with the roles swapped: up to 128 TOKENS are the M operand
//             (a TMEM lane is a token), 128 gate rows and the 128 up rows of the same
//             features lie one after the other in shared memory as ONE N operand of 256,
//             so the accumulator's columns c and c + 128 are gate and up of feature c in
//             the same lane.  An MMA of N = 256 reads 12 KB of shared memory in 128
//             cycles where two of N = 128 read 16 KB, the port's limit; a thread's GLU
//             results are consecutive features of its token and leave as 16-byte stores.
//             For busy experts (the M tile is always 128 rows).  Measured with 256 experts
//             of real width, against TC_GLU2: 933 against 929 us at 128 rows per expert,
//             1,385 against 1,533 us at 256, 2,478 against 2,528 us at 512; with 64 experts
//             and 512 rows each 619 against 701 us.  Every form moves about 13.2 TB/s from
//             L2 into shared memory there (48 KB per k-block of a tile): that is the bound.
//             Running an expert's short last tile weight-major (N as narrow as its rows) in
//             the same kernel was measured and is slower, not faster: a tile costs its
//             bytes, not its products.
//   TC_TOK    no GLU, token-major like TC_GLUT: up to 128 tokens are the M operand, 256
//             weight rows (two boxes of 128) the N operand, 256 output features per tile.
//             A thread of the epilogue owns a token and writes 16 consecutive features
//             with two 16-byte stores; with the weights as the M operand (TC_PLAIN,
//             TC_WIDE) it owns a feature and writes one 2-byte value per token, and at 256
//             rows per expert those stores, not the products, set the pace (measured: the
//             epilogue warps busy 90 % of the kernel's time, the MMA warp waiting for a
//             free accumulator 28 % of it; without the stores the kernel ran 1.67 times
//             as fast).
// (A variant with gate and up rows side by side in ONE accumulator of up to 256 tokens -
// an MMA of N = 256 reads less of A per flop from shared memory than two of N = 128 -
// was built and measured: 642 instead of 392 us at 256 rows per expert; its epilogue,
// which pairs TMEM lane f with lane f + 64 through shared memory, does not hide under
// the main loop.)
enum { TC_GLU2 = 0, TC_PLAIN = 1, TC_WIDE = 2, TC_GLUT = 3, TC_TOK = 4 };

// Persistent: one CTA per SM walks the tiles t = blockIdx.x, + gridDim.x, ...
// of the (token tile, weight tile) space, weight tile fastest, so CTAs that run
// side by side share an expert.  The TMA ring never drains between tiles and the
// accumulator is double-buffered in TMEM, so the epilogue of one tile runs under
// the main loop of the next.  The token rows come through one of four tensor maps
// with boxes of 64, 128, 192 or 256 rows: the smallest that holds the tile.
template <int MODE>
__global__ void __launch_bounds__(192) moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                          const __grid_constant__ CUtensorMap tm_x0,
                                                          const __grid_constant__ CUtensorMap tm_x1,
                                                          const __grid_constant__ CUtensorMap tm_x2,
                                                          const __grid_constant__ CUtensorMap tm_x3,
                                                          TcArgs a) {
  constexpr bool GLU2 = MODE == TC_GLU2, GLUT = MODE == TC_GLUT, GLU = GLU2 || GLUT;
  constexpr bool TOK = MODE == TC_TOK;                // token-major without GLU
  constexpr bool TMAJ = GLUT || TOK;                  // tokens are the M operand
  constexpr bool WIDE = MODE == TC_WIDE;
  // a stage holds KSUB 64-wide k-blocks: one with two weight boxes per k-block or wide
  // token boxes, two otherwise, so that every stage moves 40-48 KB and the per-stage
  // barrier round trip is paid half as often on the narrow down projection
  constexpr int TC_B_BYTES = (WIDE ? 2 : 1) * TC_MAXN * TC_BK * 2;   // reserved per k-block
  constexpr int KSUB = MODE == TC_PLAIN ? 2 : 1;
  constexpr int NA = (GLU || TOK) ? 2 : 1;                   // 16 KB weight regions per k-block
  constexpr int STAGES = MODE == TC_PLAIN ? 3 : 4;
  constexpr int STAGE_BYTES = KSUB * (NA * TC_A_BYTES + TC_B_BYTES);
  constexpr int FEAT = TOK ? 2 * TC_BM : TC_BM;       // output features per tile
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  __shared__ volatile int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntok = a.ntok;
  const int acc_cols = TMAJ ? 2 * TC_BM : (GLU2 ? 2 * ntok : ntok);   // columns of one accumulator buffer
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
  const int kblocks = (a.K + KSUB * TC_BK - 1) / (KSUB * TC_BK);
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
        // the token box: the smallest of 64 / 128 / 192 / 256 rows that holds the tile
        const int bucket = (cur.z + 63) / 64 - 1;
        const CUtensorMap* tm_x = bucket == 0 ? &tm_x0 : (bucket == 1 ? &tm_x1 : (bucket == 2 ? &tm_x2 : &tm_x3));
        const unsigned tx = KSUB * (NA * TC_A_BYTES + (unsigned)(bucket + 1) * 64 * TC_BK * 2);
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
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            // a k-block past K is all zero fill and still counts its bytes
            unsigned char* st = tiles + (size_t)s * STAGE_BYTES + sub * (NA * TC_A_BYTES + TC_B_BYTES);
            const int k = (kb * KSUB + sub) * TC_BK;
            tma_load_3d(st, &tm_w, k, n0, e, &full_bar[s]);
            if (GLU) tma_load_3d(st + TC_A_BYTES, &tm_w, k, a.n_out + n0, e, &full_bar[s]);
            if (TOK) tma_load_3d(st + TC_A_BYTES, &tm_w, k, n0 + TC_BM, e, &full_bar[s]);
            tma_load_2d(st + NA * TC_A_BYTES, tm_x, k, row0, &full_bar[s]);
          }
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
        // instruction descriptor: D f32, A/B bf16, both K-major, M = 128, N = the rows
        // this tile really has, rounded up to 16: a tile costs what it holds
        const int n_tile = cur.z;
        // (token-major GLU: M = 128 token rows, N = 256 weight rows, whatever the tile holds)
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
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const unsigned st = smem_u32(tiles + (size_t)s * STAGE_BYTES + sub * (NA * TC_A_BYTES + TC_B_BYTES));
            const unsigned sb = st + NA * TC_A_BYTES;
#pragma unroll
            for (int kk = 0; kk < TC_BK / 16; ++kk) {
              const unsigned acc = (kb | sub | kk) != 0;
              const unsigned long long bdesc = sw128_desc(sb + kk * 32);
              if (TMAJ) {                  // A: the token rows; B: two boxes of weight rows, 256 in all
                tc_mma(tmem_d, bdesc, sw128_desc(st + kk * 32), idesc, acc);
                continue;
              }
              tc_mma(tmem_d, sw128_desc(st + kk * 32), bdesc, idesc, acc);
              if (GLU2) tc_mma(tmem_d + ntok, sw128_desc(st + TC_A_BYTES + kk * 32), bdesc, idesc, acc);
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
    // epilogue: TMEM lane = weight row; this warp may touch lanes 32*(warp%4) .. +31
    const int lane_base = (warp & 3) * 32;
    __nv_bfloat16* C = (__nv_bfloat16*)a.C;
    int local = 0;
    int4 cur = tile_at(blockIdx.x);
    for (int t = blockIdx.x; t < total && cur.x >= 0; t += gridDim.x) {
      const int4 nxt = tile_at(t + gridDim.x);
      const int row0 = cur.y, row_end = cur.w;
      const int b = local & 1;
      const int n_tile = cur.z;
      // Without GLU (the down projection) a column's output row and route weight come
      // from two dependent loads from global memory: they are fetched for the whole
      // tile before the wait on the accumulator, so that this tile's main loop hides
      // them; lane l keeps columns l, l+32, ...; handed round by shuffle.  With GLU a
      // column's output row is its sorted row and nothing is loaded.
      constexpr int NQ = (GLU || TOK) ? 1 : (WIDE ? 2 : 1) * TC_MAXN / 32;
      int my_crow[NQ];
      float my_scale[NQ];
      if (!GLU && !TOK) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int row = row0 + q * 32 + lane;
          my_crow[q] = -1;
          my_scale[q] = 1.f;
          if (q * 32 + lane < n_tile && row < row_end) {
            my_crow[q] = a.c_rows ? a.c_rows[row] : row;
            if (a.row_scale) my_scale[q] = a.row_scale[my_crow[q]];
          }
        }
      }
      bool ok = mbar_wait(&acc_full[b], (unsigned)(local >> 1) & 1u, &gave_up);
      if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_MOE_EPILOGUE); gave_up = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const unsigned tmem_d = tmem_base + (unsigned)(b * acc_cols) + ((unsigned)lane_base << 16);
      if (TMAJ) {
        // TMEM lane = token row of the tile.  GLU: columns c and c + 128 are gate and up of
        // feature n0 + c; otherwise column c is feature n0 + c, 256 of them
        const int n0 = (t % wtiles) * FEAT;
        const int row = row0 + lane_base + lane;
        const bool valid = lane_base + lane < n_tile && row < row_end;
        const int crow = valid ? (a.c_rows ? a.c_rows[row] : row) : 0;
        const float scale = valid && a.row_scale ? a.row_scale[crow] : 1.f;
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
      } else if (GLU2) {
        const int n = (t % wtiles) * TC_BM + lane_base + lane;
        for (int c0 = 0; c0 < n_tile; c0 += 16) {
          unsigned g[16], u[16];
          tc_ld16(tmem_d + (unsigned)c0, g);
          tc_ld16(tmem_d + (unsigned)(c0 + ntok), u);
          tc_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int row = row0 + c0 + c;
            if (row < row_end && n < a.n_out) {
              const int crow = a.c_rows ? a.c_rows[row] : row;
              float v = tc_glu(__uint_as_float(g[c]), __uint_as_float(u[c]), a.act, a.act_alpha, a.act_limit);
              if (a.row_scale) v *= a.row_scale[crow];
              C[(size_t)crow * a.ldc + n] = __float2bfloat16_rn(v);
            }
          }
        }
      } else {
        const int n = (t % wtiles) * TC_BM + lane_base + lane;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c0 = q * 32 + half * 16;
            if (c0 < n_tile) {
              unsigned g[16];
              tc_ld16(tmem_d + (unsigned)c0, g);
              tc_ld_wait();
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                const int crow = __shfl_sync(0xffffffffu, my_crow[q], half * 16 + c);
                const float scale = __shfl_sync(0xffffffffu, my_scale[q], half * 16 + c);
                if (crow >= 0 && n < a.n_out)
                  C[(size_t)crow * a.ldc + n] = __float2bfloat16_rn(__uint_as_float(g[c]) * scale);
              }
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

// The down projection on CTA PAIRS (`cta_group::2`): a cluster of two CTAs computes
//   D[256 weight rows, N tokens] = W_e tile * X^T,   N = 32..256 in steps of 32.
// CTA r of the pair loads weight rows n0 + 128 r .. + 127 (its half of the M operand)
// and token rows row0 + r N/2 .. (its half of the N operand) into its own shared memory;
// the even CTA issues one MMA of M = 256 per 16 k, which reads both halves of the tokens
// from both CTAs and leaves 128 accumulator rows in each CTA's TMEM.  A k-block moves
// 16 KB of weights and at most 16 KB of tokens into a CTA where a lone CTA moves 16 + 32.
//
//   full[s]       (even CTA's) counts the bytes of BOTH CTAs' loads of stage s
//   empty[s]      (each CTA's own) the even CTA's commit arrives on both
//   acc_full[b]   (each CTA's own) likewise
//   acc_empty[b]  (even CTA's) the four epilogue warps of both CTAs arrive on it
// The roles are those of the kernel above; the odd CTA's warp 1 only allocates TMEM.
// Neither CTA leaves before the other is done with its shared memory and barriers: the
// producers wait for the last commits on their stages, and a cluster barrier precedes
// the TMEM release.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = TC_A_BYTES + TC_MAXN * TC_BK * 2;   // 16 KB weights + up to 128 token rows

__global__ void __launch_bounds__(192) moe_gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                               const __grid_constant__ CUtensorMap tm_x0,
                                                               const __grid_constant__ CUtensorMap tm_x1,
                                                               const __grid_constant__ CUtensorMap tm_x2,
                                                               const __grid_constant__ CUtensorMap tm_x3,
                                                               TcArgs a) {
  constexpr int STAGES = PAIR_STAGES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  __shared__ volatile int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();          // 0: the pair's leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int ntok = a.ntok;                          // at most 256
  const unsigned tmem_cols = 512;                   // two accumulators of up to 256 columns
  if (threadIdx.x == 0) {
    gave_up = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  __syncwarp();
  cluster_sync_all();                               // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  const int kblocks = (a.K + TC_BK - 1) / TC_BK;
  const int wtiles = (a.n_out + 2 * TC_BM - 1) / (2 * TC_BM);
  const int total = a.tiles_y * wtiles;
  // (the pair's MMA covers a tile's rows rounded up to 32, so that each CTA holds a multiple
  // of 16; a role reads the entry of its next tile while it works on the current one)
  auto tile_at = [&](int t) {
    int4 ti = t < total ? __ldg(&a.tile_info[t / wtiles]) : make_int4(-1, 0, 0, 0);
    ti.z = (ti.z + 31) & ~31;
    return ti;
  };

  if (warp == 0) {
    if (lane == 0) {
      long long issued = 0;
      bool ok = true;
      const unsigned leader_full = cluster_addr_of(&full_bar[0], 0);   // + 8 s: the leader's full[s]
      int4 cur = tile_at(pair);
      for (int t = pair; t < total && ok && cur.x >= 0; t += pairs) {
        const int4 nxt = tile_at(t + pairs);
        const int n0 = (t % wtiles) * 2 * TC_BM + (int)rank * TC_BM;
        const int e = cur.x;
        const int half = cur.z >> 1;
        const int row0 = cur.y + (int)rank * half;
        // the token box: the smallest of 32 / 64 / 96 / 128 rows that holds this CTA's half
        const int bucket = (half + 31) / 32 - 1;
        const CUtensorMap* tm_x = bucket == 0 ? &tm_x0 : (bucket == 1 ? &tm_x1 : (bucket == 2 ? &tm_x2 : &tm_x3));
        const unsigned tx = 2u * (TC_A_BYTES + (unsigned)(bucket + 1) * 32 * TC_BK * 2);   // both CTAs' bytes
        for (int kb = 0; kb < kblocks; ++kb, ++issued) {
          const int s = (int)(issued % STAGES);
          const unsigned ph = (unsigned)(issued / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_MOE_PRODUCER);
            gave_up = 1;
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&full_bar[s], tx);
          unsigned char* st = tiles + (size_t)s * PAIR_STAGE_BYTES;
          const int k = kb * TC_BK;
          tma_load_3d_pair(st, &tm_w, k, n0, e, leader_full + 8u * (unsigned)s);
          tma_load_2d_pair(st + TC_A_BYTES, tm_x, k, row0, leader_full + 8u * (unsigned)s);
        }
        cur = nxt;
      }
      // the leader's commits for the last uses of the stages arrive on this CTA's barriers:
      // stay until they have (and, after a failure, until copies in flight have landed)
      for (long long kb = issued > STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
        const int s = (int)(kb % STAGES);
        const unsigned ph = (unsigned)(kb / STAGES) & 1u;
        if (!gave_up) {
          if (!mbar_wait(&empty_bar[s], ph, &gave_up)) {
            atomicCAS(a.status, 0, FT_ST_MOE_PRODUCER);
            gave_up = 1;
          }
        } else if (rank == 0) {
          const unsigned long long start = global_ns();
          while (!mbar_try(&full_bar[s], ph) && global_ns() - start < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      long long done = 0;
      int local = 0;
      bool ok = true;
      int4 cur = tile_at(pair);
      for (int t = pair; t < total && ok && cur.x >= 0; t += pairs) {
        const int4 nxt = tile_at(t + pairs);
        const int n_tile = cur.z;
        // D f32, A/B bf16, both K-major, M = 256 over the pair, N = the tile's rows
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n_tile >> 3) << 17) |
                               ((unsigned)((2 * TC_BM) >> 4) << 24);
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((unsigned)(local >> 1) & 1u) ^ 1u, &gave_up)) {
          atomicCAS(a.status, 0, FT_ST_MOE_MMA_ACC);
          gave_up = 1;
          break;
        }
        tc_fence_after();
        const unsigned tmem_d = tmem_base + (unsigned)(b * ntok);
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
          const unsigned st = smem_u32(tiles + (size_t)s * PAIR_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk)
            tc_mma_pair(tmem_d, sw128_desc(st + kk * 32), sw128_desc(st + TC_A_BYTES + kk * 32), idesc,
                        (kb | kk) != 0);
          tc_commit_pair(&empty_bar[s]);
        }
        if (ok) tc_commit_pair(&acc_full[b]);
        ++local;
        cur = nxt;
      }
    }
  } else {
    // epilogue: TMEM lane = one of this CTA's 128 weight rows
    const int lane_base = (warp & 3) * 32;
    __nv_bfloat16* C = (__nv_bfloat16*)a.C;
    unsigned leader_acc_empty[2];
    leader_acc_empty[0] = cluster_addr_of(&acc_empty[0], 0);
    leader_acc_empty[1] = cluster_addr_of(&acc_empty[1], 0);
    int local = 0;
    int4 cur = tile_at(pair);
    for (int t = pair; t < total && cur.x >= 0; t += pairs) {
      const int4 nxt = tile_at(t + pairs);
      const int row0 = cur.y, row_end = cur.w;
      const int b = local & 1;
      const int n_tile = cur.z;
      // a column's output row and route weight, fetched before the accumulator is waited
      // for; lane l keeps columns l, l + 32, ...; handed round by shuffle
      constexpr int NQ = 2 * TC_MAXN / 32;
      int my_crow[NQ];
      float my_scale[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const int row = row0 + q * 32 + lane;
        my_crow[q] = -1;
        my_scale[q] = 1.f;
        if (q * 32 + lane < n_tile && row < row_end) {
          my_crow[q] = a.c_rows ? a.c_rows[row] : row;
          if (a.row_scale) my_scale[q] = a.row_scale[my_crow[q]];
        }
      }
      bool ok = mbar_wait(&acc_full[b], (unsigned)(local >> 1) & 1u, &gave_up);
      if (!ok && lane == 0) { atomicCAS(a.status, 0, FT_ST_MOE_EPILOGUE); gave_up = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const unsigned tmem_d = tmem_base + (unsigned)(b * ntok) + ((unsigned)lane_base << 16);
      const int n = (t % wtiles) * 2 * TC_BM + (int)rank * TC_BM + lane_base + lane;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c0 = q * 32 + half * 16;
          if (c0 < n_tile) {
            unsigned g[16];
            tc_ld16(tmem_d + (unsigned)c0, g);
            tc_ld_wait();
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const int crow = __shfl_sync(0xffffffffu, my_crow[q], half * 16 + c);
              const float scale = __shfl_sync(0xffffffffu, my_scale[q], half * 16 + c);
              if (crow >= 0 && n < a.n_out)
                C[(size_t)crow * a.ldc + n] = __float2bfloat16_rn(__uint_as_float(g[c]) * scale);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty[b]);
      ++local;
      cur = nxt;
    }
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
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
  moe_gemm_tc_kernel<MODE><<<grid, 192, smem, stream>>>(mw, mx[0], mx[1], mx[2], mx[3], a);
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

// `map_w`: the 3-D map of the expert weights with boxes of 128 rows.  `maps_x`: four 2-D
// maps of the sorted token rows, 128 bytes each, with boxes of 64, 128, 192 and 256 rows.
// `ntok`: most rows of a token tile (a multiple of 16; up to 128 with GLU, else up to 256).
// `glu`: 0 none; 1 gate and up as two accumulators, weights as the M operand; 2 tokens as
// the M operand and gate + up rows as one N operand of 256; 3 no GLU, tokens as the M
// operand and 256 weight rows as the N operand (`ntok` at most 128 for 1 to 3).
int ft_moe_gemm_tc(const void* map_w, const void* maps_x, void* C, long long ldc,
                   const int* group_offsets, const int* active, const void* tile_info, const int* c_rows,
                   const float* row_scale, int* status, int rows_bound, int n_out, int K, int G,
                   int ntok, int glu, int act, float act_alpha, float act_limit,
                   cudaStream_t stream) {
  if (rows_bound <= 0 || n_out <= 0) return FT_OK;
  if (ntok < 16 || ntok > ((glu == 1 || glu == 2 || glu == 3) ? TC_MAXN : 2 * TC_MAXN) || (ntok & 15) || (K & 7) ||
      G <= 0 || glu < 0 || glu > 3)
    return FT_ERR_SHAPE;
  CUtensorMap mw, mx[4];
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(mx, maps_x, sizeof(mx));
  const int tiles_y = ft_tc_tiles_bound(rows_bound, G, ntok);
  TcArgs a{C, group_offsets, active, (const int4*)tile_info, c_rows, row_scale, status, ldc, n_out, K, G, ntok,
           tiles_y, act, act_alpha, act_limit};
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int feat = glu == 3 ? 2 * TC_BM : TC_BM;
  const int total = tiles_y * ((n_out + feat - 1) / feat);
  dim3 grid(total < sms ? total : sms);
  constexpr int B_BYTES = TC_MAXN * TC_BK * 2;
  int rc;
  if (glu == 3) rc = launch_tc<TC_TOK>(mw, mx, a, grid, 4 * (2 * TC_A_BYTES + B_BYTES) + 1024, stream);
  else if (glu == 2) rc = launch_tc<TC_GLUT>(mw, mx, a, grid, 4 * (2 * TC_A_BYTES + B_BYTES) + 1024, stream);
  else if (glu) rc = launch_tc<TC_GLU2>(mw, mx, a, grid, 4 * (2 * TC_A_BYTES + B_BYTES) + 1024, stream);
  else if (ntok > TC_MAXN) rc = launch_tc<TC_WIDE>(mw, mx, a, grid, 4 * (TC_A_BYTES + 2 * B_BYTES) + 1024, stream);
  else rc = launch_tc<TC_PLAIN>(mw, mx, a, grid, 3 * 2 * (TC_A_BYTES + B_BYTES) + 1024, stream);
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

// The down projection (no GLU) on CTA pairs: `maps_x` holds four 2-D maps of the sorted
// token rows with boxes of 32, 64, 96 and 128 rows (a CTA loads half of a tile's rows);
// `ntok` (a multiple of 32, at most 256) and the tile map as for ft_moe_gemm_tc.
int ft_moe_gemm_tc_pair(const void* map_w, const void* maps_x, void* C, long long ldc,
                        const int* group_offsets, const int* active, const void* tile_info,
                        const int* c_rows, const float* row_scale, int* status,
                        int rows_bound, int n_out, int K, int G, int ntok, cudaStream_t stream) {
  if (rows_bound <= 0 || n_out <= 0) return FT_OK;
  if (ntok < 32 || ntok > 2 * TC_MAXN || (ntok & 31) || (K & 7) || G <= 0) return FT_ERR_SHAPE;
  CUtensorMap mw, mx[4];
  memcpy(&mw, map_w, sizeof(mw));
  memcpy(mx, maps_x, sizeof(mx));
  const int tiles_y = ft_tc_tiles_bound(rows_bound, G, ntok);
  TcArgs a{C, group_offsets, active, (const int4*)tile_info, c_rows, row_scale, status, ldc, n_out, K, G, ntok,
           tiles_y, 0, 0.f, 0.f};
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int total = tiles_y * ((n_out + 2 * TC_BM - 1) / (2 * TC_BM));
  const int pairs = total < sms / 2 ? total : sms / 2;
  const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, moe_gemm_tc_pair_kernel, mw, mx[0], mx[1], mx[2], mx[3], a);
  if (e != cudaSuccess) return (int)e;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
