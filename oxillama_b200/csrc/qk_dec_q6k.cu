// Instantiates the decode kernels of one format (policy qkdec::DecQ6K, qk_dec_fmts.cuh).
#include "qk_dec_fmts.cuh"

QK_DEC_DEFINE(q6k, qkdec::DecQ6K)
