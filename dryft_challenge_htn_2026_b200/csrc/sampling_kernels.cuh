// Device code of the sampler (see sampling.cu for the rule it implements): the counter hash, the
// two kernels (per-chunk partial argmax, merge of a row's chunks) and their chunk size. Shared by
// the entry points in sampling.cu and sample_noalloc.cu.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7FEB352Du;
    x ^= x >> 15;
    x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}

__device__ __forceinline__ float gumbel(uint32_t seed_lo, uint32_t seed_hi, uint32_t pos, uint32_t idx) {
    uint32_t x = mix32(idx ^ 0x9E3779B9u);
    x = mix32(x + pos * 0x85EBCA6Bu + seed_lo);
    x = mix32(x ^ seed_hi);
    const float u = ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
    return -logf(-logf(u));
}

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

#define SAMPLE_CHUNK 4096

// grid (chunks, rows). Row b reads logits[b * V ...]; its position is pos[rows ? rows[b] : b] + 1
// (the place the new token will take); position < 0 marks a padding row.
__global__ void sample_partial_kernel(const float* logits, int V, const float* temperature,
                                      const uint32_t* seeds, const int* pos, const int* rows,
                                      float* ws_val, int* ws_idx) {
    __shared__ float sv[32];
    __shared__ int si[32];
    // temperatures and seeds are not written by the kernel before this one: they are fetched before
    // the wait for it. The position is read after the wait, with the logits: the kernel before may be
    // the one that advances it (two calls back to back on the same positions).
    const int b = blockIdx.y, chunk = blockIdx.x;
    const float temp = temperature[b];
    const uint32_t s_lo = seeds[2 * b], s_hi = seeds[2 * b + 1];
    const int pos_at = rows ? rows[b] : b;
    pdl_wait();
    pdl_launch_dependents();
    const float* row = logits + (size_t)b * V;
    const int begin = chunk * SAMPLE_CHUNK, end = min(V, begin + SAMPLE_CHUNK);
    float bv = -INFINITY;
    int bi = begin;
    // 16 logits a thread as four 16-byte loads where the rows are 16-byte aligned
    const bool wide = V % 4 == 0 && blockDim.x * 16 == SAMPLE_CHUNK && ((uintptr_t)logits & 15) == 0;
    float4 z4[4];
    if (wide) {   // requested together, and together with the position, before any is looked at
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int i = begin + (k * (int)blockDim.x + (int)threadIdx.x) * 4;
            z4[k] = i < end ? *reinterpret_cast<const float4*>(row + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
    }
    const int p = pos[pos_at];
    if (p >= 0) {
        const float inv_t = temp > 0.f ? 1.f / temp : 1.f;
        if (wide) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = begin + (k * (int)blockDim.x + (int)threadIdx.x) * 4;
                const float z[4] = {z4[k].x, z4[k].y, z4[k].z, z4[k].w};
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (i + e < end) {
                        float v = z[e];
                        if (temp > 0.f) v = v * inv_t + gumbel(s_lo, s_hi, (uint32_t)(p + 1), (uint32_t)(i + e));
                        better(bv, bi, v, i + e);
                    }
            }
        } else {
            for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
                float z = row[i];
                if (temp > 0.f) z = z * inv_t + gumbel(s_lo, s_hi, (uint32_t)(p + 1), (uint32_t)i);
                better(bv, bi, z, i);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            better(bv, bi, ov, oi);
        }
        if (lane == 0) {
            ws_val[(size_t)b * gridDim.x + chunk] = bv;
            ws_idx[(size_t)b * gridDim.x + chunk] = bi;
        }
    }
}

// One warp per row merges the chunks, writes the token, and (advance != 0) moves the row's
// position on by one so that the next decode step of a captured graph finds it in place.
__global__ void sample_final_kernel(const float* ws_val, const int* ws_idx, int chunks, int* pos, const int* rows,
                                    int* out_tok, int advance) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x, lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < chunks; c += 32) better(bv, bi, ws_val[(size_t)b * chunks + c], ws_idx[(size_t)b * chunks + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
    if (lane == 0) {
        const int r = rows ? rows[b] : b;
        const int p = pos[r];
        out_tok[b] = (p >= 0 && bi != 0x7fffffff) ? bi : 0;
        if (advance && p >= 0) pos[r] = p + 1;
    }
}
