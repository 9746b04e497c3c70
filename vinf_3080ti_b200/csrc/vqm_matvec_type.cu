// One translation unit per GGUF type (-DVQM_TYPE=<id> -DVQM_TYPE_NAME=<name>): instantiates the matvec
// kernel for M = 1..8 activation rows and the row-group heights the launcher picks from, and exports one
// launcher.  Splitting by type keeps the build parallel.
#include "vqm_matvec.cuh"

#ifndef VQM_TYPE
#error "compile with -DVQM_TYPE=<GGUF type id> -DVQM_TYPE_NAME=<name>"
#endif

namespace vqm {
namespace {

// Rows a warp takes per chunk: 8 for one or two activation rows (more independent work per staged
// activation load), 4 beyond that (registers), 2 where eight-row stages of a wide type do not fit.
template <int M>
constexpr int rows_per_chunk() {
    constexpr int want = M <= 2 ? 8 : 4;
    return matvec_smem_bytes_for<VQM_TYPE, want, M>() <= 100 * 1024 ? want
         : matvec_smem_bytes_for<VQM_TYPE, want / 2, M>() <= 200 * 1024 ? want / 2 : want / 4;
}

template <int M>
cudaError_t launch_one(const MatvecArgs &a, int sm_count, cudaStream_t stream, int *grid_out) {
    constexpr int RW = rows_per_chunk<M>();
    constexpr size_t smem = matvec_smem_bytes_for<VQM_TYPE, RW, M>();
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
    // one wave; a short tensor gets fewer blocks so that every warp still has a row
    int grid = sm_count * blocks_per_sm;
    const int want = (a.rows + kWarps - 1) / kWarps;
    if (grid > want) grid = want;
    if (grid_out != nullptr) *grid_out = grid;
    qmv_kernel<VQM_TYPE, M, RW><<<grid, kWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

#define VQM_CAT2(a, b) a##b
#define VQM_CAT(a, b) VQM_CAT2(a, b)

cudaError_t VQM_CAT(launch_qmv_, VQM_TYPE_NAME)(const MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid_out) {
    switch (m) {
        case 1: return launch_one<1>(a, sm_count, stream, grid_out);
        case 2: return launch_one<2>(a, sm_count, stream, grid_out);
        case 3: return launch_one<3>(a, sm_count, stream, grid_out);
        case 4: return launch_one<4>(a, sm_count, stream, grid_out);
        case 5: return launch_one<5>(a, sm_count, stream, grid_out);
        case 6: return launch_one<6>(a, sm_count, stream, grid_out);
        case 7: return launch_one<7>(a, sm_count, stream, grid_out);
        case 8: return launch_one<8>(a, sm_count, stream, grid_out);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace vqm
