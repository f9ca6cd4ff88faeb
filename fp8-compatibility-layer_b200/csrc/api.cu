// Library-level entry points of the C ABI: version, per-thread error text, device status word.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace tfp8b {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return TFP8B_ERR_CUDA;
}

int read_and_clear_status(unsigned int* word_on_device, unsigned int* out, cudaStream_t st) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, word_on_device, sizeof(v), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && v) e = cudaMemsetAsync(word_on_device, 0, sizeof(v), st);
    if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
    *out |= v;
    return TFP8B_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides_bytes, const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TFP8B_ERR_CUDA; }
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r)); return TFP8B_ERR_CUDA; }
    return TFP8B_OK;
}

int gemv_status(unsigned int* out, cudaStream_t st);
int gemm_status(unsigned int* out, cudaStream_t st);
int glue_status(unsigned int* out, cudaStream_t st);
int gemm_mx_status(unsigned int* out, cudaStream_t st);

}  // namespace tfp8b

using namespace tfp8b;

extern "C" int tfp8b_version(void) { return TFP8B_VERSION; }

extern "C" const char* tfp8b_last_error_string(void) { return t_error; }

extern "C" int tfp8b_device_status(unsigned int* out_status, tfp8b_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int v = 0;
    int rc = gemv_status(&v, st);
    if (rc == TFP8B_OK) rc = gemm_status(&v, st);
    if (rc == TFP8B_OK) rc = glue_status(&v, st);
    if (rc == TFP8B_OK) rc = gemm_mx_status(&v, st);
    if (rc != TFP8B_OK) return rc;
    if (out_status) *out_status = v;
    if (v) {
        set_error("a kernel reported a problem (status 0x%x:%s%s%s%s)", v, (v & STATUS_GEMV_WAIT) ? " gemv wait ran out;" : "",
                  (v & STATUS_GEMM_WAIT) ? " gemm wait ran out;" : "",
                  (v & STATUS_GLUE_WAIT) ? " all-reduce: a peer never answered, the rows were set to NaN;" : "",
                  (v & STATUS_GLUE_POS) ? " rope_kv_store: a position outside the KV cache was skipped;" : "");
        return TFP8B_ERR_DEVICE;
    }
    return TFP8B_OK;
}
