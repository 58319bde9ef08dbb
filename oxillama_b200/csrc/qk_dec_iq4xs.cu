// Instantiates the decode kernels of one format (policy qkdec::DecIQ4XS, qk_dec_fmts.cuh).
#include "qk_dec_fmts.cuh"

QK_DEC_DEFINE(iq4xs, qkdec::DecIQ4XS)
