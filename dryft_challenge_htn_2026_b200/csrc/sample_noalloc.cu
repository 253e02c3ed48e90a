// The sampler without caller-provided scratch: see sample_noalloc.h for who needs it and the rules.
// Same kernels as dk_sample (sampling_kernels.cuh); their partial results go to a fixed device
// array of this file instead of memory the caller allocated.
#include "sample_noalloc.h"
#include "sampling_kernels.cuh"

// First half: the per-chunk best values (float), second half: their indices (int).
static __device__ __align__(256) unsigned char dk_noalloc_scratch[DK_NOALLOC_SCRATCH_BYTES];

#define DK_NOALLOC_MAX_DEVICES 64
// Device address of the array on each GPU. In host code the array's name is only a handle for the
// runtime, not an address a kernel could use, so the address is asked for once per device.
static void* g_scratch_addr[DK_NOALLOC_MAX_DEVICES];

static int scratch_for_current_device(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= DK_NOALLOC_MAX_DEVICES) return DK_NOALLOC_BAD_ARGUMENT;
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, dk_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

DK_EXPORT const char* dk_sample_noalloc_error(int code) {
    if (code == 0) return "no error";
    if (code == DK_NOALLOC_TOO_LARGE)
        return "dk_sample_noalloc: n_rows * ceil(V / 4096) exceeds the 16384 partial results the built-in scratch holds";
    if (code == DK_NOALLOC_BAD_ARGUMENT) return "dk_sample_noalloc: bad argument (null pointer, size < 1, or device index)";
    return cudaGetErrorString((cudaError_t)code);
}

DK_EXPORT int dk_sample_noalloc(const float* logits, int n_rows, int V, const float* temperature, const uint32_t* seeds,
                                int* pos, const int* rows, int* out_tok, int advance, cudaStream_t stream) {
    if (!logits || !temperature || !seeds || !pos || !out_tok || n_rows < 1 || V < 1) return DK_NOALLOC_BAD_ARGUMENT;
    const long long chunks = ((long long)V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    if (chunks * n_rows > DK_NOALLOC_MAX_PARTIALS) return DK_NOALLOC_TOO_LARGE;
    void* base = nullptr;
    int e = scratch_for_current_device(&base);
    if (e) return e;
    float* ws_val = reinterpret_cast<float*>(base);
    int* ws_idx = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + DK_NOALLOC_MAX_PARTIALS * sizeof(float));
    e = dk_launch(sample_partial_kernel, dim3((unsigned)chunks, n_rows), dim3(256), 0, stream, logits, V, temperature,
                  seeds, (const int*)pos, rows, ws_val, ws_idx);
    if (e) return e;
    return dk_launch(sample_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)ws_val, (const int*)ws_idx,
                     (int)chunks, pos, rows, out_tok, advance);
}
