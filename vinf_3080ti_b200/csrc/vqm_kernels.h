// Host-visible declarations shared by the kernel translation units and the runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace vqm {

constexpr int kMaxParts = 4;  // tensors one launch can cover (they share the activations, the type and the columns)

// Row-sharded matvec across GPUs: where a launch stores its outputs inside every rank's exchange region (plain remote
// stores over NVLink, issued by the lane that holds the output) and which flags order that against the consumers.
struct PushInfo {
    unsigned long long region[8];  // device address of every rank's exchange region, this rank's included
    unsigned *pushes;              // this rank's own count of pushes per slot, unsigned[n_slots] (inside its region)
    long long dst_off[kMaxParts];  // per tensor: byte offset, inside a region, of its gathered y[0][0]
    long long flag_off;            // byte offset, inside a region, of the flag table: unsigned flags[slot][8 ranks], the
                                   // number of pushes of the slot each rank has completed
    int n_ranks, rank;
    int rows_total[kMaxParts];     // per tensor: the gathered tensor has rows_total rows ...
    int row_begin[kMaxParts];      // ... and this rank's slice starts at row_begin
    int push_slot;                 // 1 + flag slot signalled after the push (0: no push)
    int wait_slot;                 // 1 + slot every rank must have pushed as often as this rank before x is read (0: no wait)
};

// One tensor of a launch.  The launch numbers the rows of its tensors consecutively; tensor p owns launch rows
// [row_end of tensor p - 1, row_end).  Unused entries have row_end = INT_MAX.
struct MatvecPart {
    const uint8_t *w;  // raw blocks, readable up to 15 bytes past the end
    float *y;          // [M][rows] fp32 (may be null when only the argmax is wanted)
    int row_end;
    int rows;          // rows of this tensor (the stride of y)
};

struct MatvecArgs {
    MatvecPart part[kMaxParts];
    const float *x;          // [M][cols] fp32, 16-byte aligned
    const uint8_t *codebook;  // device copy of the type's GGUF codebook (IQ2/IQ3 types), else null
    unsigned *status;        // device error word (0 = fine)
    // fused argmax (all null / 0 when unused; single-tensor launches only)
    float *part_val;         // [kMaxTok][gridDim.x]
    int *part_idx;           // [kMaxTok][gridDim.x]
    unsigned *done_counter;  // zero before the launch; the kernel leaves it zero
    int *out_idx;            // [M] winning row (+ row_base), 0x7fffffff if the column has no value above -inf
    float *out_val;          // [M] winning value (may be null)
    int rows, cols;          // rows: of all tensors together
    long long row_bytes;
    int row_base;            // added to row numbers reported by the argmax (row-sharded weights)
    // Column split for short launches: the k_split blocks of a thread-block cluster share a group of rows (one row per
    // warp), each takes a range of the column segments and leaves its partial sums in the shared memory of the
    // cluster's first block, which adds them in the order of k and writes the outputs.
    int k_split;             // chosen by the launcher (from the rows and the columns only, never from M); 1 = off
    int allow_split;         // host only: the caller permits the split
    int overlap_launch;      // host only: launch with programmatic stream serialization (see qmv_kernel)
    int max_grid;            // host only: upper bound on the grid (0 = none); sizes the argmax partial arrays
    // Fused prologue / epilogue (the flags of the reference's megakernel QMV, engine/csrc/common/qwen_mk_abi.h:55-58):
    //   kFuseSiluMul: the activations are silu(x) * x2;  kFuseNorm: then rmsnorm over the columns times norm_w;
    //   kFuseAdd: y += W x instead of y = W x (the outputs already hold the residual).
    int fuse;                // kFuse* bits, 0 = plain matvec
    const float *x2;         // [M][cols], with kFuseSiluMul
    const float *norm_w;     // [cols], with kFuseNorm
    float eps;               // rmsnorm epsilon
    PushInfo push;           // all zero when the tensor is not sharded
};

enum : int { kFuseAdd = 1, kFuseNorm = 2, kFuseSiluMul = 8 };  // (4 is the fused argmax, which has its own fields)

constexpr int kMaxSplit = 8;  // column ranges a row can be split into (the portable cluster size)

enum : unsigned { kStatusOk = 0, kStatusWaitExpired = 1, kStatusPeerWaitExpired = 2 };

// One launcher per GGUF type (vqm_matvec_type.cu).  m: activation rows (1..8); sm_count: SMs of the device;
// grid_out (optional) receives the grid size used.
#define VQM_FOR_EACH_TYPE(X) \
    X(0, F32) X(1, F16) X(8, Q8_0) X(10, Q2_K) X(11, Q3_K) X(12, Q4_K) X(13, Q5_K) X(14, Q6_K) X(16, IQ2_XXS) \
    X(17, IQ2_XS) X(18, IQ3_XXS) X(20, IQ4_NL) X(21, IQ3_S) X(22, IQ2_S) X(23, IQ4_XS)
#define VQM_DECLARE_LAUNCHER(id, name)                                                                            \
    cudaError_t launch_qmv_##name(const MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid_out); \
    cudaError_t launch_qmv_fused_##name(const MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid_out);  // honours a.fuse
VQM_FOR_EACH_TYPE(VQM_DECLARE_LAUNCHER)
#undef VQM_DECLARE_LAUNCHER

constexpr int kMaxGrid = 4096;  // upper bound on the matvec grid (sizes the argmax partial arrays)

// Prompt-pass GEMM on the tensor cores (vqm_gemm.cu).  xh: fp16 activations [ntok padded to gemm_token_tile()][cols].
int gemm_token_tile();
cudaError_t launch_f32_to_f16_rows(const float *x, void *xh, long long n_valid, long long n_total, cudaStream_t stream);
cudaError_t launch_qgemm(int type, const uint8_t *w, const void *xh, float *y, int rows, int cols, long long row_bytes, int ntok,
                         const uint8_t *codebook, cudaStream_t stream);

// Prompt-pass GEMM on tcgen05 tensor cores with the accumulators in tensor memory (vqm_gemm_tc5.cu): xh padded to
// gemm_tc5_token_tile() rows; needs cols to be a multiple of 64.  status: device word that receives a code if a bounded
// wait expires.
int gemm_tc5_token_tile();
bool gemm_tc5_supports(int cols);
cudaError_t launch_qgemm_tc5(int type, const uint8_t *w, const void *xh, float *y, int rows, int cols, long long row_bytes, int ntok,
                             const uint8_t *codebook, unsigned *status, cudaStream_t stream);

cudaError_t launch_argmax_rows(const float *x, int n, int ntok, int *out, cudaStream_t stream);
cudaError_t launch_dequant(int type, const uint8_t *w, float *out, long long numel, const uint8_t *codebook,
                           cudaStream_t stream);

}  // namespace vqm
