// The single translation unit of liblme_cuda.so: every kernel file is included here so that the device status
// word and the helpers are shared without relocatable device code.
#include "kernels/gemm.cu"
#include "kernels/gemm2cta.cu"
#include "kernels/elementwise.cu"
#include "kernels/fp8.cu"
#include "kernels/moe.cu"
#include "kernels/conv1d.cu"
#include "kernels/ssd.cu"
#include "kernels/m2rnn.cu"
#include "kernels/rnn.cu"
#include "kernels/rows.cu"
#include "kernels/attention.cu"
#include "kernels/noalloc.cu"
