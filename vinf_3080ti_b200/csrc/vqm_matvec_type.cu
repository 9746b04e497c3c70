// One translation unit per GGUF type (-DVQM_TYPE=<id> -DVQM_TYPE_NAME=<name>): instantiates the matvec
// kernel for M = 1..8 activation rows and the row-group heights the launcher picks from, and exports one
// launcher.  Splitting by type keeps the build parallel.
#include "vqm_matvec.cuh"

#ifndef VQM_TYPE
#error "compile with -DVQM_TYPE=<GGUF type id> -DVQM_TYPE_NAME=<name>"
#endif

namespace vqm {
namespace {

// One kernel per (activation rows M, rows per chunk RW).  A warp always decodes RW rows per chunk (rows that do not
// exist are computed and dropped), so RW is chosen per launch: the smallest height that covers a warp's share of
// the rows, up to 4 (registers, and RW * M <= 32 outputs per warp).
template <int M, int RW>
struct Variant {
    static constexpr size_t kSmem = matvec_smem_bytes_for<VQM_TYPE, RW, M>();
    static constexpr bool kFits = kSmem <= 200 * 1024 && RW * M <= 32;

    // blocks per SM (cached; one device per process), 0 if the variant cannot run
    static int blocks_per_sm() {
        static int cached = -1;
        if (cached >= 0) return cached;
        cached = 0;
        if constexpr (kFits) {
            if (cudaFuncSetAttribute(qmv_kernel<VQM_TYPE, M, RW, kFusedBuild>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kSmem)) == cudaSuccess) {
                int n = 0;
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, qmv_kernel<VQM_TYPE, M, RW, kFusedBuild>, kWarps * 32, kSmem) == cudaSuccess)
                    cached = n;
            }
            (void)cudaGetLastError();
        }
        return cached;
    }

    // rows each warp would get in a one-wave launch (rounded up), or 0 if the variant cannot run
    static int rows_per_warp(int rows, int sm_count) {
        const int b = blocks_per_sm();
        if (b == 0) return 0;
        const int warps = grid_for(rows, sm_count, b) * kWarps;
        return (rows + warps - 1) / warps;
    }

    static int grid_for(int rows, int sm_count, int b) {
        // one wave; a short tensor gets fewer blocks so that every warp still has a row
        const int grid = sm_count * b, want = (rows + kWarps - 1) / kWarps;
        return grid < want ? grid : want;
    }

    static cudaError_t launch(const MatvecArgs &a, int sm_count, cudaStream_t stream, int *grid_out) {
        if constexpr (kFits) {
            int grid = grid_for(a.rows, sm_count, blocks_per_sm());
            if (a.k_split > 1) grid = (a.rows + kWarps - 1) / kWarps * a.k_split;  // one row per warp, k_split blocks per group
            if (a.max_grid > 0 && grid > a.max_grid) grid = a.max_grid;
            if (grid_out != nullptr) *grid_out = grid;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(grid);
            cfg.blockDim = dim3(kWarps * 32);
            cfg.dynamicSmemBytes = kSmem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[2];
            int n_attr = 0;
            if (a.overlap_launch) {
                attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
                ++n_attr;
            }
            if (a.k_split > 1) {  // the blocks that share a group of rows form a cluster
                attr[n_attr].id = cudaLaunchAttributeClusterDimension;
                attr[n_attr].val.clusterDim.x = static_cast<unsigned>(a.k_split);
                attr[n_attr].val.clusterDim.y = 1;
                attr[n_attr].val.clusterDim.z = 1;
                ++n_attr;
            }
            cfg.attrs = attr;
            cfg.numAttrs = n_attr;
            return cudaLaunchKernelEx(&cfg, qmv_kernel<VQM_TYPE, M, RW, kFusedBuild>, a);
        } else {
            return cudaErrorInvalidConfiguration;
        }
    }
};

// Column split for short launches.  When the rows cover less than half of the warps a full grid has (two blocks per SM
// of kWarps warps - a nominal figure, so that the choice never depends on M and an M-row pass stays equal to M
// single-row passes bit for bit), every row goes to one warp of a group and k blocks per group share the columns
// (evenly, in units of 256): k = warps / rows, at most kMaxSplit (a portable cluster) and at most one block per unit.
inline int choose_split(const MatvecArgs &a, int sm_count) {
    if (!a.allow_split || a.out_idx != nullptr) return 1;
    const int warps = sm_count * 2 * kWarps, n_units = (a.cols + 255) / 256;
    if (a.rows * 2 > warps) return 1;
    int k = warps / a.rows;
    if (k > kMaxSplit) k = kMaxSplit;
    if (k > n_units) k = n_units;
    return k;
}

template <int M>
cudaError_t launch_one(const MatvecArgs &args, int sm_count, cudaStream_t stream, int *grid_out) {
    MatvecArgs a = args;
    a.k_split = choose_split(a, sm_count);
    if (a.k_split > 1) return Variant<M, 1>::launch(a, sm_count, stream, grid_out);
    // Taller chunks cost a block per SM (shared memory) and more than they save.  (Two-row chunks at two blocks per SM
    // for more than 4 activation rows were measured too: slower, 106 instead of 74 us for Q4_K 17408 x 5120 at M = 8.)
    // smallest RW that holds a warp's share; the tallest (4) if the share needs several chunks anyway
    if (const int n = Variant<M, 1>::rows_per_warp(a.rows, sm_count); n > 0 && n <= 1) return Variant<M, 1>::launch(a, sm_count, stream, grid_out);
    if (const int n = Variant<M, 2>::rows_per_warp(a.rows, sm_count); n > 0 && n <= 2) return Variant<M, 2>::launch(a, sm_count, stream, grid_out);
    if (Variant<M, 4>::blocks_per_sm() > 0) return Variant<M, 4>::launch(a, sm_count, stream, grid_out);
    if (Variant<M, 2>::blocks_per_sm() > 0) return Variant<M, 2>::launch(a, sm_count, stream, grid_out);
    return Variant<M, 1>::launch(a, sm_count, stream, grid_out);
}

}  // namespace

#define VQM_CAT2(a, b) a##b
#define VQM_CAT(a, b) VQM_CAT2(a, b)

#if VQM_FUSED
#define VQM_LAUNCHER_PREFIX launch_qmv_fused_
#else
#define VQM_LAUNCHER_PREFIX launch_qmv_
#endif

cudaError_t VQM_CAT(VQM_LAUNCHER_PREFIX, VQM_TYPE_NAME)(const MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid_out) {
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
