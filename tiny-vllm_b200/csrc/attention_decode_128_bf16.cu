// The fused decode attention for head size 128 and bfloat16 norm weights: one of six libraries made of
// attention_decode_body.cuh, so that a model compiles the combination it uses and no other.
#include "common.cuh"

#define TVB_DECODE_HEAD_DIM 128
#define TVB_DECODE_WEIGHT bf16
#include "attention_decode_body.cuh"
