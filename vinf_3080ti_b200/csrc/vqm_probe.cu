// Instruction issue rates of this GPU's SMs for the instruction kinds the matvec decoders are made of.
//
// The matvec kernels are bound by instruction issue, not by HBM; how many scheduler cycles a byte permute, a logic op, a
// packed FMA or the whole decode sequence of 8 weights costs is what their roofline rests on.  This probe measures it
// on the device it runs on: one block per SM, `warps` warps per block, every thread runs kIter iterations of 16
// independent instructions of one kind (or of a fixed mix) between two clock64() reads.  Reported: scheduler cycles
// per warp instruction (an SM has four schedulers; warps / 4 of the block's warps share one).
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/vinf_b200.h"

namespace {

constexpr int kIter = 2048;
using f32x2 = unsigned long long;

#define P_FMA2(d, a, b, c) asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c))
#define P_PRMT(d, a, s) asm volatile("prmt.b32 %0, %1, 0, %2;" : "=r"(d) : "r"(a), "n"(s))
#define P_AND(d, a, m) asm volatile("and.b32 %0, %1, %2;" : "=r"(d) : "r"(a), "n"(m))
#define P_PACK(d, a, b) asm volatile("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(a), "r"(b))

// kind: 0 PRMT, 1 LOP3, 2 FFMA2, 3 FFMA, 4 IMAD, 5 SHF, 6 cvt.f32.f16, 7 PRMT and FFMA2 alternating,
//       8 / 9 the decode sequence of 8 packed 4-bit weights of one row (ld.shared, 2 and, 8 prmt, 4 packed FMAs field ->
//       weight, 4 packed FMAs per activation row) with 1 / 4 activation rows: result in cycles per 8 weights.
template <int KIND>
__global__ void __launch_bounds__(1024) probe_kernel(unsigned *sink, long long *cycles, uint32_t seed) {
    __shared__ uint32_t words[4096];
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) words[i] = i * seed;
    __syncthreads();
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(words)) + (threadIdx.x & 31) * 4;
    uint32_t r[16];
    f32x2 q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        r[i] = seed * (i + 1) + threadIdx.x;
        q[i] = (static_cast<unsigned long long>(r[i]) * 0x100000001ull) | 0x3f0000003f000000ull;
    }
    const f32x2 one = 0x3f8000003f800000ull, dl = one + seed, nl = one ^ 0x100000001ull;
    constexpr int NT = KIND == 9 ? 4 : 1;
    const long long t0 = clock64();
#pragma unroll 1
    for (int it = 0; it < kIter; ++it) {
        if constexpr (KIND == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("prmt.b32 %0, %0, %1, 0x4404;" : "+r"(r[i]) : "r"(seed));
        } else if constexpr (KIND == 1) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("and.b32 %0, %0, %1;" : "+r"(r[i]) : "r"(seed));
        } else if constexpr (KIND == 2) {
#pragma unroll
            for (int i = 0; i < 16; ++i) P_FMA2(q[i], q[i], one, q[i]);
        } else if constexpr (KIND == 3) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("fma.rn.f32 %0, %0, %1, %0;" : "+r"(r[i]) : "r"(0x3f800000u));
        } else if constexpr (KIND == 4) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("mad.lo.u32 %0, %0, %1, %0;" : "+r"(r[i]) : "r"(seed));
        } else if constexpr (KIND == 5) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("shr.b32 %0, %0, %1;" : "+r"(r[i]) : "r"(seed & 3u));
        } else if constexpr (KIND == 6) {
#pragma unroll
            for (int i = 0; i < 16; ++i) asm volatile("{ .reg .b16 t; mov.b32 {t, _}, %0; cvt.f32.f16 %0, t; }" : "+r"(r[i]));
        } else if constexpr (KIND == 7) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                asm volatile("prmt.b32 %0, %0, %1, 0x4404;" : "+r"(r[i]) : "r"(seed));
                P_FMA2(q[i], q[i], one, q[i]);
            }
        } else {
            uint32_t w[4];
#pragma unroll
            for (int row = 0; row < 4; ++row) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[row]) : "r"(base + ((it & 31) * 4 + row) * 128));
#pragma unroll
            for (int row = 0; row < 4; ++row) {
                uint32_t lo, hi, p[8];
                P_AND(lo, w[row], 0x0F0F0F0F);
                P_AND(hi, w[row], 0xF0F0F0F0);
                P_PRMT(p[0], lo, 0x4404); P_PRMT(p[1], lo, 0x4414); P_PRMT(p[2], lo, 0x4424); P_PRMT(p[3], lo, 0x4434);
                P_PRMT(p[4], hi, 0x4404); P_PRMT(p[5], hi, 0x4414); P_PRMT(p[6], hi, 0x4424); P_PRMT(p[7], hi, 0x4434);
                f32x2 a0, a1, b0, b1;
                P_PACK(a0, p[0], p[1]); P_PACK(a1, p[2], p[3]); P_PACK(b0, p[4], p[5]); P_PACK(b1, p[6], p[7]);
                P_FMA2(a0, a0, dl, nl); P_FMA2(a1, a1, dl, nl); P_FMA2(b0, b0, dl, nl); P_FMA2(b1, b1, dl, nl);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    P_FMA2(q[row * 4 + t], a0, q[(row * 4 + t + 1) & 15], q[row * 4 + t]);
                    P_FMA2(q[row * 4 + t], a1, one, q[row * 4 + t]);
                    P_FMA2(q[row * 4 + t], b0, dl, q[row * 4 + t]);
                    P_FMA2(q[row * 4 + t], b1, nl, q[row * 4 + t]);
                }
            }
        }
    }
    const long long t1 = clock64();
    unsigned acc = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc ^= r[i] ^ static_cast<unsigned>(q[i]) ^ static_cast<unsigned>(q[i] >> 32);
    sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cycles = t1 - t0;
}

template <int KIND>
cudaError_t run_one(int sm_count, int warps, unsigned *sink, long long *cycles_dev, double *out) {
    for (int rep = 0; rep < 2; ++rep) probe_kernel<KIND><<<sm_count, warps * 32>>>(sink, cycles_dev, 3u);
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return err;
    long long cycles = 0;
    err = cudaMemcpy(&cycles, cycles_dev, sizeof(cycles), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return err;
    // per scheduler: warps / 4 warps, each kIter x (16 instructions | 4 units of 8 weights)
    const double per_iter = KIND >= 8 ? 4.0 : 16.0;
    *out = static_cast<double>(cycles) / (static_cast<double>(kIter) * per_iter * (warps / 4.0));
    return cudaSuccess;
}

}  // namespace

extern "C" int vqm_probe_issue_rates(int warps_per_sm, double *out, int n) {
    if (out == nullptr || n < VQM_PROBE_KINDS) return 2;                                   // VQM_ERR_VALUE
    if (warps_per_sm < 4 || warps_per_sm > 32 || warps_per_sm % 4 != 0) return 2;
    int dev = 0, sm_count = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    unsigned *sink = nullptr;
    long long *cycles = nullptr;
    if (err == cudaSuccess) err = cudaMalloc(&sink, static_cast<size_t>(sm_count) * 1024 * sizeof(unsigned));
    if (err == cudaSuccess) err = cudaMalloc(&cycles, sizeof(long long));
    if (err == cudaSuccess) err = run_one<0>(sm_count, warps_per_sm, sink, cycles, out + 0);
    if (err == cudaSuccess) err = run_one<1>(sm_count, warps_per_sm, sink, cycles, out + 1);
    if (err == cudaSuccess) err = run_one<2>(sm_count, warps_per_sm, sink, cycles, out + 2);
    if (err == cudaSuccess) err = run_one<3>(sm_count, warps_per_sm, sink, cycles, out + 3);
    if (err == cudaSuccess) err = run_one<4>(sm_count, warps_per_sm, sink, cycles, out + 4);
    if (err == cudaSuccess) err = run_one<5>(sm_count, warps_per_sm, sink, cycles, out + 5);
    if (err == cudaSuccess) err = run_one<6>(sm_count, warps_per_sm, sink, cycles, out + 6);
    if (err == cudaSuccess) err = run_one<7>(sm_count, warps_per_sm, sink, cycles, out + 7);
    if (err == cudaSuccess) err = run_one<8>(sm_count, warps_per_sm, sink, cycles, out + 8);
    if (err == cudaSuccess) err = run_one<9>(sm_count, warps_per_sm, sink, cycles, out + 9);
    cudaFree(sink);
    cudaFree(cycles);
    return err == cudaSuccess ? 0 : 5;  // VQM_OK / VQM_ERR_CUDA
}
