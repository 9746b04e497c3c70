// Small kernels beside the matvec: row argmax over a logits buffer and the exact dequantiser.
#include "vqm_formats.cuh"
#include "vqm_kernels.h"

namespace vqm {
namespace {

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// Row t of x ([ntok][n]) -> out[t].  Same result as the reference's argmax_kernel
// (engine/csrc/megakernel/qwen_runtime.cu:851-876): the maximum under a strict '>' scan from -inf, the lowest
// index among equal maxima, 0x7fffffff when no element is above -inf (all -inf or NaN).
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *x_all, int n, int *out_all) {
    const float *x = x_all + static_cast<size_t>(blockIdx.x) * n;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (v > bv) {  // indices only grow within a thread, so '>' keeps the lowest
            bv = v;
            bi = i;
        }
    }
    __shared__ float s_v[32];
    __shared__ int s_i[32];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? s_v[lane] : -INFINITY;
        bi = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out_all[blockIdx.x] = bi;
    }
}

// One thread per 8-weight chunk; blocks are read straight from global memory.
template <int TYPE>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *w, float *out, long long n_chunks, const uint8_t *codebook) {
    __shared__ __align__(16) uint8_t table[grid_bytes(TYPE) > 0 ? grid_bytes(TYPE) : 16];
    if constexpr (grid_bytes(TYPE) > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x)
                reinterpret_cast<uint32_t *>(table)[i] = reinterpret_cast<const uint32_t *>(codebook)[i];
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
        __syncthreads();
    }
    constexpr int CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_chunks;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float v[8];
        deq8<TYPE>(w + (i / CPB) * BB, static_cast<int>(i % CPB), v, table);
        float4 *o = reinterpret_cast<float4 *>(out + i * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

template <int TYPE>
cudaError_t launch_dequant_t(const uint8_t *w, float *out, long long numel, const uint8_t *codebook, cudaStream_t stream) {
    const long long n_chunks = numel / 8;
    long long blocks = (n_chunks + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    dequant_kernel<TYPE><<<static_cast<int>(blocks), 256, 0, stream>>>(w, out, n_chunks, codebook);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_argmax_rows(const float *x, int n, int ntok, int *out, cudaStream_t stream) {
    argmax_rows_kernel<<<ntok, 1024, 0, stream>>>(x, n, out);
    return cudaGetLastError();
}

cudaError_t launch_dequant(int type, const uint8_t *w, float *out, long long numel, const uint8_t *codebook,
                           cudaStream_t stream) {
    switch (type) {
        case kF32: return launch_dequant_t<kF32>(w, out, numel, codebook, stream);
        case kF16: return launch_dequant_t<kF16>(w, out, numel, codebook, stream);
        case kQ8_0: return launch_dequant_t<kQ8_0>(w, out, numel, codebook, stream);
        case kQ2_K: return launch_dequant_t<kQ2_K>(w, out, numel, codebook, stream);
        case kQ3_K: return launch_dequant_t<kQ3_K>(w, out, numel, codebook, stream);
        case kQ4_K: return launch_dequant_t<kQ4_K>(w, out, numel, codebook, stream);
        case kQ5_K: return launch_dequant_t<kQ5_K>(w, out, numel, codebook, stream);
        case kQ6_K: return launch_dequant_t<kQ6_K>(w, out, numel, codebook, stream);
        case kIQ4_NL: return launch_dequant_t<kIQ4_NL>(w, out, numel, codebook, stream);
        case kIQ3_S: return launch_dequant_t<kIQ3_S>(w, out, numel, codebook, stream);
        case kIQ4_XS: return launch_dequant_t<kIQ4_XS>(w, out, numel, codebook, stream);
        case kIQ2_XXS: return launch_dequant_t<kIQ2_XXS>(w, out, numel, codebook, stream);
        case kIQ2_XS: return launch_dequant_t<kIQ2_XS>(w, out, numel, codebook, stream);
        case kIQ2_S: return launch_dequant_t<kIQ2_S>(w, out, numel, codebook, stream);
        case kIQ3_XXS: return launch_dequant_t<kIQ3_XXS>(w, out, numel, codebook, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace vqm
