// Dequant-fused GEMM for many activation rows on the 5th-generation tensor cores (tcgen05, TMEM).
// Interface of gemm_tc.cu; see there for the design.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

constexpr int TC_COLS = 64;            // activation rows (GEMM columns) per launch
constexpr int TC_MIN_ROWS = 9;         // fewer rows than this stay on the GEMV kernels

// Can this problem run on the tcgen05 path?  (STORE / GEGLU / SWIGLU epilogues, 9..64 rows.)
bool gemm_tc_supports(int wtype, const GemvArgs& a);
// Allocates the path's workspace (outside any stream capture).  Idempotent; false when out of memory.
bool gemm_tc_prepare();
void gemm_tc_release();
// Enqueues the row-quantisation kernel and the GEMM.  Returns ADAMAH_OK or an error code.
int launch_gemm_tc(int wtype, const GemvArgs& a, cudaStream_t stream);

}  // namespace ab
