// Instantiates the decode kernels of one format (policy qkdec::DecQ40, qk_dec_fmts.cuh).
#include "qk_dec_fmts.cuh"

QK_DEC_DEFINE(q40, qkdec::DecQ40)
