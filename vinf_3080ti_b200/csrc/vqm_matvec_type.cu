// One translation unit per GGUF type (-DVQM_TYPE=<id> -DVQM_TYPE_NAME=<name>): instantiates the matvec
// kernel for M = 1..8 activation rows and the row-group heights the launcher picks from, and exports one
// launcher.  Splitting by type keeps the build parallel.
#include "vqm_matvec.cuh"

#ifndef VQM_TYPE
#error "compile with -DVQM_TYPE=<GGUF type id> -DVQM_TYPE_NAME=<name>"
#endif

namespace vqm {
namespace {

template <int M, int RW>
cudaError_t launch_one(const MatvecArgs &a, int sm_count, cudaStream_t stream, int *grid_out) {
    constexpr size_t smem = matvec_smem_bytes(VQM_TYPE, RW);
    static int blocks_per_sm = 0;  // one device per process
    if (blocks_per_sm == 0) {
        cudaError_t err = cudaFuncSetAttribute(qmv_kernel<VQM_TYPE, M, RW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess) return err;
        int n = 0;
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, qmv_kernel<VQM_TYPE, M, RW>, kWarps * 32, smem);
        if (err != cudaSuccess) return err;
        blocks_per_sm = n > 0 ? n : 1;
    }
    const int n_rg = (a.rows + RW - 1) / RW;
    int grid = sm_count * blocks_per_sm;
    if (grid > n_rg) grid = n_rg;
    if (grid_out != nullptr) *grid_out = grid;
    qmv_kernel<VQM_TYPE, M, RW><<<grid, kWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int RW>
cudaError_t launch_m(const MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid_out) {
    switch (m) {
        case 1: return launch_one<1, RW>(a, sm_count, stream, grid_out);
        case 2: return launch_one<2, RW>(a, sm_count, stream, grid_out);
        case 3: return launch_one<3, RW>(a, sm_count, stream, grid_out);
        case 4: return launch_one<4, RW>(a, sm_count, stream, grid_out);
        case 5: return launch_one<5, RW>(a, sm_count, stream, grid_out);
        case 6: return launch_one<6, RW>(a, sm_count, stream, grid_out);
        case 7: return launch_one<7, RW>(a, sm_count, stream, grid_out);
        case 8: return launch_one<8, RW>(a, sm_count, stream, grid_out);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

#define VQM_CAT2(a, b) a##b
#define VQM_CAT(a, b) VQM_CAT2(a, b)

// rw: rows per warp row group (2 or 4; wide unquantised rows only fit 2).
cudaError_t VQM_CAT(launch_qmv_, VQM_TYPE_NAME)(const MatvecArgs &a, int m, int rw, int sm_count, cudaStream_t stream,
                                                int *grid_out) {
    if (rw >= 4 && matvec_smem_bytes(VQM_TYPE, 4) <= 200 * 1024) return launch_m<4>(a, m, sm_count, stream, grid_out);
    return launch_m<2>(a, m, sm_count, stream, grid_out);
}

}  // namespace vqm
