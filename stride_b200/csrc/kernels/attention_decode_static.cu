// The allocation-free variant of decode attention declared in
// attention_decode_static.h: the kernel of attention_decode.cu in its cp.async
// form (the TMA form needs a status word and the cache's extent, which this
// entry point does not take), with the partial results of the key splits kept
// in an array that is part of this library's device image instead of a buffer
// the caller allocates.
#include "attention_decode_static.h"

#include "attention_decode.cu"   // the kernels and their launcher; nothing there is changed

// Device storage for the partial results. In host code this name is only a
// handle for cudaGetSymbolAddress; it is not a pointer a kernel may be given.
static __device__ __align__(256) float g_decode_static_scratch[STRIDE_DECODE_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};      // per device, filled on the first call there

// Looks up (once per device, with that device current) where the array lives on the device.
int scratch_for_current_device(float** address) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (device < 0 || device >= kMaxDevices) return STRIDE_BAD_ARGUMENT;
    if (g_scratch_address[device] == nullptr) {
        // This may be the first CUDA call the library makes: bind its runtime to the
        // device that is current, so that the library's device image can be found.
        e = cudaSetDevice(device);
        if (e != cudaSuccess) return static_cast<int>(e);
        float* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_static_scratch);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (p == nullptr) return STRIDE_BAD_ARGUMENT;
        g_scratch_address[device] = p;
    }
    *address = g_scratch_address[device];
    return 0;
}

}  // namespace

extern "C" {

long long stride_paged_decode_attention_static_floats(int tokens, int nq, int nkv, int hd, int max_context) {
    return stride_paged_decode_scratch_floats(tokens, nq, nkv, hd, max_context);
}

int stride_paged_decode_attention_static(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                         const int32_t* block_table, int table_width, const int32_t* seq_of_token,
                                         const int32_t* positions, int tokens, int nq, int nkv, int hd, int page_size,
                                         float scale, int window, int max_context, cudaStream_t stream) {
    if (tokens < 0 || nq <= 0 || nkv <= 0 || max_context <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const long long need = stride_paged_decode_scratch_floats(tokens, nq, nkv, hd, max_context);
    if (need > STRIDE_DECODE_STATIC_SCRATCH_FLOATS) return STRIDE_STATIC_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    // From here on this is the ordinary entry point, fed the static array.
    return stride_paged_decode_attention(q, q_stride, out, k_pages, v_pages, block_table, table_width, seq_of_token, positions,
                                         scratch, STRIDE_DECODE_STATIC_SCRATCH_FLOATS, tokens, nq, nkv, hd, page_size, scale,
                                         window, max_context, stream);
}

}  // extern "C"
