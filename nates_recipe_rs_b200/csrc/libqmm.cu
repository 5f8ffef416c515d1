// Single translation unit of libqmm: the kernels share one device status word
// and are compiled without relocatable device code.
#include "api.cu"
#include "quantize.cu"
#include "qmatvec.cu"
#include "qmatvec_jobs.cu"
#include "qgemm.cu"
#include "qmatvec_mma.cu"
#include "decoder_ops.cu"
#include "tp_comm.cu"
#include "attn_entry.cu"
#include "ops_entry.cu"
#include "gguf.cu"
#include "decoder.cu"
