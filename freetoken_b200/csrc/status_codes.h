// Codes a kernel leaves in the device status word when one of its bounded
// waits ran out: which kernel, and which of its roles gave up.  The word holds
// the FIRST failure since it was last cleared (atomicCAS from 0).  This table
// is the only place the numbers live: the kernels use the FT_ST_* names, and
// the Python side reads the X(...) lines of this file to turn a code into a
// message.
#pragma once

// X(name, code, kernel, role)
#define FT_STATUS_TABLE(X)                                                              \
  X(MOE_PRODUCER, 1, "moe_gemm_tc", "the TMA producer (a free stage of the ring)")      \
  X(MOE_MMA_STAGE, 2, "moe_gemm_tc", "the MMA issuer (a filled stage of the ring)")     \
  X(MOE_EPILOGUE, 3, "moe_gemm_tc", "the epilogue warps (a finished accumulator)")      \
  X(MOE_MMA_ACC, 4, "moe_gemm_tc", "the MMA issuer (a drained accumulator)")            \
  X(PREFILL_PRODUCER, 11, "attn_prefill_tc", "the TMA producer (a free K or V stage)")  \
  X(PREFILL_MMA_Q, 12, "attn_prefill_tc", "the MMA issuer (the query tile)")            \
  X(PREFILL_MMA_K, 13, "attn_prefill_tc", "the MMA issuer (a K tile)")                  \
  X(PREFILL_MMA_PV, 14, "attn_prefill_tc", "the MMA issuer (P, a V tile or its cleaning)") \
  X(PREFILL_SOFTMAX_S, 15, "attn_prefill_tc", "the softmax warps (a score tile)")       \
  X(PREFILL_SOFTMAX_PV, 16, "attn_prefill_tc", "the softmax warps (the previous P.V product)") \
  X(PREFILL_SOFTMAX_LAST, 17, "attn_prefill_tc", "the softmax warps (the last P.V product)") \
  X(PREFILL_CLEANER, 19, "attn_prefill_tc", "the warp that zeroes stale V rows (the last V tile)") \
  X(DECODE_PRODUCER, 21, "attn_decode_tma", "the TMA producer (a free stage)")          \
  X(DECODE_CONSUMER, 22, "attn_decode_tma", "the consumer warps (a filled stage)")      \
  X(SELFTEST_WAIT, 31, "wait_selftest", "the waiting thread (a barrier nobody arrives at)")

#define FT_STATUS_ENUM_ENTRY(name, code, kernel, role) FT_ST_##name = code,
enum FtStatusCode { FT_STATUS_TABLE(FT_STATUS_ENUM_ENTRY) FT_ST_END };
