// The weight-streaming product for 1 to 8 rows of x: one of four libraries made of
// gemm_small_m_body.cuh, so that a decode step compiles the templates of its own batch size only.
#define TVB_SMALL_M_NT 1
#include "gemm_small_m_body.cuh"
