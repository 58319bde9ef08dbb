// Instantiates the decode kernels of one format (policy qkdec::DecQ80, qk_dec_fmts.cuh).
#include "qk_dec_fmts.cuh"

QK_DEC_DEFINE(q80, qkdec::DecQ80)
