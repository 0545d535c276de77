// The weight-streaming product for 25 to 32 rows of x: one of four libraries made of
// gemm_small_m_body.cuh, so that a decode step compiles the templates of its own batch size only.
#define TVB_SMALL_M_NT 4
#include "gemm_small_m_body.cuh"
