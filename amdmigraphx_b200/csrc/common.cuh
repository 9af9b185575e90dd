// Host-side helpers shared by the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>
#include "../../include/mgx_cuda.h"

namespace mgx {

typedef CUresult (*cuTensorMapEncodeTiled_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                             const cuuint64_t*, const cuuint64_t*,
                                             const cuuint32_t*, const cuuint32_t*,
                                             CUtensorMapInterleave, CUtensorMapSwizzle,
                                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled obtained through the runtime (no link-time dependency
// on libcuda); nullptr when the driver does not provide it.
cuTensorMapEncodeTiled_t get_tensor_map_encoder();

// Number of SMs of the current device (cached per device).
int device_sm_count();

// Opt a kernel in to `bytes` of dynamic shared memory on the current device,
// once per (kernel, device).
int ensure_smem_optin(const void* kernel, int bytes);

// dst[b][c][r] = src[b][r][c] for 8-bit elements; src dense [rows, cols], dst row
// stride ld_dst >= rows (padding bytes are left untouched).
int transpose_8bit_ld(const void* src, void* dst, int64_t rows, int64_t cols, int64_t batch,
                      int64_t ld_dst, cudaStream_t stream);
int transpose_16bit_ld(const void* src, void* dst, int64_t rows, int64_t cols, int64_t batch,
                       int64_t ld_dst, cudaStream_t stream);

// Status words of the translation units that own bounded waits.
int qgemm_status(unsigned int* out);
int w4a16_status(unsigned int* out);
int w4a16_tc_status(unsigned int* out);
int w4a16_prefill_status(unsigned int* out);
int qgemv_status(unsigned int* out);

// skinny-M quant_dot (qgemv.cu)
bool qgemv_applicable(const mgx_qgemm_desc& d, bool has_residual, bool has_qout);
size_t qgemv_workspace(const mgx_qgemm_desc& d);
int qgemv_launch(const mgx_qgemm_desc& d, const void* A, const void* B, void* D, const float* scale,
                 const float* bias, int64_t ldb, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream);

// tcgen05 int4 prefill path (w4a16_prefill.cu)
bool w4a16_prefill_applicable(const mgx_w4_desc& d, const void* A, const void* Bp);
int w4a16_prefill_launch(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                         const void* zp, void* D, cudaStream_t stream);

// tcgen05 int4 decode path (w4a16_tc.cu)
bool w4a16_tc_applicable(const mgx_w4_desc& d);
bool w4a16_tc_pointers_ok(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                          const void* zp);
size_t w4a16_tc_workspace(const mgx_w4_desc& d);
int w4a16_tc_launch(const mgx_w4_desc& d, const void* A, const void* Bp, const void* scales,
                    const void* zp, void* D, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

} // namespace mgx
