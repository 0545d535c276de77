// The fused decode attention for head size 256 and float32 norm weights: one of six libraries made of
// attention_decode_body.cuh, so that a model compiles the combination it uses and no other.
#include "common.cuh"

#define TVB_DECODE_HEAD_DIM 256
#define TVB_DECODE_WEIGHT float
#include "attention_decode_body.cuh"
