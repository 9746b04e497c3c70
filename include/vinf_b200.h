/* vinf_b200.h - C ABI of the B200 (sm_100a) quantized-matvec engine.
 *
 * Drop-in for the quantized matvec path of the reference's CPython type `vinf._cuda_qwen_runtime.Runtime`
 * (engine/csrc/megakernel/qwen_runtime.cu:2602-2704): named weight tensors kept in raw GGUF block layout in
 * device memory, named fp32 device buffers, y = W x for 1..8 (or more) activation rows, row argmax, and the
 * fused LM-head matvec + argmax.  Each entry point names the reference method it replaces.
 *
 * Conventions
 *   - Every function returns a vqm_status.  On failure vqm_last_error() gives a message; the status maps
 *     1:1 onto the Python exception the reference raises (KeyError, ValueError, TypeError, MemoryError,
 *     RuntimeError for CUDA errors - engine/csrc/megakernel/qwen_runtime.cu:1100-1103).
 *   - All kernels and asynchronous copies of a runtime go to ONE stream owned by the runtime
 *     (vqm_stream()).  It is a blocking stream, so it also orders against work that another library
 *     in the same process puts on the legacy default stream, which is where the reference launches.
 *   - qmv / copy / zero are asynchronous; write / read / matvec / argmax* block, like the reference.
 *   - One host thread drives a runtime at a time (the reference holds the GIL in every method).
 *   - Weights are always resident in device memory: there is no host staging ring.
 */
#ifndef VINF_B200_H
#define VINF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vqm_runtime vqm_runtime;

typedef enum vqm_status {
    VQM_OK = 0,
    VQM_ERR_KEY = 1,    /* unknown tensor / buffer name            -> KeyError     */
    VQM_ERR_VALUE = 2,  /* bad type id, shape, size, offset, ntok  -> ValueError   */
    VQM_ERR_TYPE = 3,   /* fp16 buffer where fp32 is required      -> TypeError    */
    VQM_ERR_MEMORY = 4, /* device allocation failed                -> MemoryError  */
    VQM_ERR_CUDA = 5    /* any other CUDA failure, or a kernel's bounded wait expired -> RuntimeError */
} vqm_status;

/* GGUF tensor type ids accepted by vqm_upload (engine/csrc/common/qwen_quant.cuh:17-33). */
enum {
    VQM_F32 = 0, VQM_F16 = 1, VQM_Q8_0 = 8, VQM_Q2_K = 10, VQM_Q3_K = 11, VQM_Q4_K = 12, VQM_Q5_K = 13,
    VQM_Q6_K = 14, VQM_IQ2_XXS = 16, VQM_IQ2_XS = 17, VQM_IQ3_XXS = 18, VQM_IQ4_NL = 20, VQM_IQ3_S = 21,
    VQM_IQ2_S = 22, VQM_IQ4_XS = 23
};

typedef struct vqm_tensor_info_t {
    uint64_t addr; /* device address of the raw blocks */
    int32_t type, rows, cols;
    int64_t row_bytes, nbytes;
    int32_t resident; /* always 1 */
} vqm_tensor_info_t;

/* Message of the most recent failing call on this thread (never NULL). */
const char *vqm_last_error(void);

/* Runtime(iq3s_grid) - engine/csrc/megakernel/qwen_runtime.cu:1272-1297.  iq3s_grid: the 512 x 4 byte IQ3_S
 * codebook (2048 bytes), or NULL to leave it unset.  Uses the current CUDA device. */
int vqm_runtime_create(const void *iq3s_grid, size_t nbytes, vqm_runtime **out);
/* tp_dealloc - qwen_runtime.cu:1299-1336: frees every tensor and buffer the runtime owns. */
void vqm_runtime_destroy(vqm_runtime *rt);

/* Codebooks of the other IQ types: "iq2xxs_grid" (2048 B), "iq2xs_grid" (4096), "iq2s_grid" (8192),
 * "iq3xxs_grid" (1024), "iq3s_grid" (2048).  The reference compiles the first four in
 * (engine/csrc/common/qwen_iq_tables.h) and takes IQ3_S's from the caller; here the caller supplies all. */
int vqm_set_codebook(vqm_runtime *rt, const char *name, const void *data, size_t nbytes);

/* upload(name, data, type, cols, rows[, resident, group]) - qwen_runtime.cu:1338-1409.  Synchronous copy of
 * raw blocks; re-upload replaces; the allocation is padded by 16 bytes and rounded up to 256. */
int vqm_upload(vqm_runtime *rt, const char *name, const void *data, size_t nbytes, int type, int cols, int rows);
/* free(name) / has(name) / device_bytes() - qwen_runtime.cu:1411-1432 */
int vqm_free(vqm_runtime *rt, const char *name);
int vqm_has(vqm_runtime *rt, const char *name, int *out);
int vqm_device_bytes(vqm_runtime *rt, size_t *out);
/* tensor_info(name) - qwen_runtime.cu:1458-1471 */
int vqm_tensor_info(vqm_runtime *rt, const char *name, vqm_tensor_info_t *out);

/* alloc(name, n[, elem]) - qwen_runtime.cu:1616-1650: zero-filled buffer of n elements of 4 (fp32) or 2 bytes. */
int vqm_alloc(vqm_runtime *rt, const char *name, size_t n, int elem);
/* Registers caller-owned device memory under a buffer name (the runtime will not free it).  Lets a second
 * runtime or a torch tensor share memory, the use the reference makes of buffer_ptr (qwen_runtime.cu:1473-1483). */
int vqm_bind(vqm_runtime *rt, const char *name, void *device_ptr, size_t n, int elem);
/* Weights straight from a file: `nbytes` raw block bytes at byte `offset` of `path` (for a GGUF file: the tensor's
 * absolute offset) become the resident tensor `name`, without passing through a caller buffer.  Replaces the reference's
 * mmap + blocking upload per tensor (engine/src/vinf/cuda/qwen_runtime.py:68-86 over GGUFFile.mmap_tensor,
 * engine/src/vinf/gguf/parser.py:153-159).  `threads` (1..16, 0 = 4) readers pread 8 MiB chunks into pinned staging and
 * copy them to the device on their own streams, so reading and copying overlap.  Synchronous; same shape checks and
 * errors as vqm_upload, plus VQM_ERR_VALUE when the file cannot be opened, is too short or a read fails. */
int vqm_upload_file(vqm_runtime *rt, const char *name, const char *path, uint64_t offset, uint64_t nbytes, int type, int cols, int rows,
                    int threads);
/* Same for a weight tensor that already sits in device memory (e.g. a row shard of a larger tensor). */
int vqm_bind_tensor(vqm_runtime *rt, const char *name, const void *device_ptr, int type, int cols, int rows);
int vqm_release(vqm_runtime *rt, const char *buffer_name);
/* write(name, bytes[, offset]) / read(name[, n, offset]) - qwen_runtime.cu:1819-1858; offsets in elements. */
int vqm_write(vqm_runtime *rt, const char *name, const void *data, size_t nbytes, size_t offset);
int vqm_read(vqm_runtime *rt, const char *name, void *out, size_t n, size_t offset);
/* copy(dst, dst_off, src, src_off, n) - qwen_runtime.cu:2200-2217; zero(name) - :1652-1667; zero_range - :2589-2600 */
int vqm_copy(vqm_runtime *rt, const char *dst, size_t dst_off, const char *src, size_t src_off, size_t n);
int vqm_zero(vqm_runtime *rt, const char *name);
int vqm_zero_range(vqm_runtime *rt, const char *name, size_t offset, size_t n);
/* buffer_ptr(name) -> (addr, n) - qwen_runtime.cu:1473-1483; buffer_elem(name) - :2317-2322 */
int vqm_buffer_ptr(vqm_runtime *rt, const char *name, uint64_t *addr, size_t *n);
int vqm_buffer_elem(vqm_runtime *rt, const char *name, int *elem);
/* Element count of a buffer of either precision (what read(name) with n = -1 returns). */
int vqm_buffer_len(vqm_runtime *rt, const char *name, size_t *n);
int vqm_buffer_bytes(vqm_runtime *rt, size_t *out);

/* qmv(weight, x, y[, ntok]) - qwen_runtime.cu:1861-1912: y[t][r] = sum_k W[r][k] x[t][k], x = [ntok][cols],
 * y = [ntok][rows], both fp32 buffers.  Asynchronous.  More than 8 rows run as groups of 8. */
int vqm_qmv(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok);
/* matvec(name, x) -> y - qwen_runtime.cu:2281-2315: synchronous single-row entry with host vectors. */
int vqm_matvec(vqm_runtime *rt, const char *weight, const float *x_host, size_t x_bytes, float *y_host, size_t y_bytes);
/* argmax(x, n) / argmax_rows(x, n, ntok) - qwen_runtime.cu:2167-2197: blocking; ties to the lowest index;
 * 1 <= ntok <= 256. */
int vqm_argmax(vqm_runtime *rt, const char *x, int n, int *out);
int vqm_argmax_rows(vqm_runtime *rt, const char *x, int n, int ntok, int *out);
/* The LM head in one launch: qmv(weight, x, y, ntok) followed by argmax_rows(y, rows, ntok)
 * (engine/src/vinf/qwen_gpu.py:1068-1086; the reference fuses the two only in its megakernel,
 * engine/csrc/megakernel/qwen_megakernel.cu:231-236,800-829).  y may be NULL to skip storing the logits.
 * ntok <= 8.  out_ids (host, ntok ints) may be NULL: then the call is asynchronous and the ids stay in
 * the device buffer returned by vqm_argmax_result(). */
int vqm_qmv_argmax(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int *out_ids);
/* The matvec with the prologues and epilogues of the reference's fused QMV instruction (flags and meaning:
 * engine/csrc/common/qwen_mk_abi.h:55-58, engine/csrc/megakernel/qwen_megakernel.cu:486-550 and :231), so that the
 * element-wise kernels around a matvec need no launch of their own:
 *   VQM_FUSE_SILU_MUL  the activations are silu(x) * x2 (the FFN's down projection reads gate and up directly);
 *   VQM_FUSE_NORM      then v * rsqrt(mean(v^2) + eps) * norm_weight over the columns of each activation row
 *                      (norm_weight: an fp32 buffer of `cols` values, or an F32 tensor with `cols` elements);
 *   VQM_FUSE_ADD       y += W v instead of y = W v (y already holds the residual);
 *   VQM_FUSE_ARGMAX    the fused argmax of vqm_qmv_argmax over the stored values (after the residual); out_ids as there.
 * 1 <= ntok <= 8; every activation row is transformed on its own.  x and x2 are not modified. */
enum { VQM_FUSE_ADD = 1, VQM_FUSE_NORM = 2, VQM_FUSE_ARGMAX = 4, VQM_FUSE_SILU_MUL = 8 };
int vqm_qmv_fused(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int flags, const char *x2,
                  const char *norm_weight, float eps, int *out_ids);
/* Device arrays holding the last fused argmax: ids[8] (int32) and values[8] (fp32). */
int vqm_argmax_result(vqm_runtime *rt, uint64_t *ids_addr, uint64_t *values_addr);
/* Blocking copy of the first ntok ids (and, if values is not NULL, values) of the last fused argmax to the host. */
int vqm_argmax_fetch(vqm_runtime *rt, int ntok, int *ids, float *values);
/* Row offset added to the ids of the fused argmax (for a runtime that holds rows [base, base + rows) of a
 * row-sharded LM head). */
int vqm_set_argmax_row_base(vqm_runtime *rt, const char *weight, int row_base);

/* Exact fp32 values of a weight tensor into an fp32 buffer of rows * cols elements.  No reference method;
 * exposes the block decoders the matvec uses so that they can be checked bit for bit against the
 * reference dequantiser (engine/src/vinf/gguf/dequant.py:17-57). */
int vqm_dequantize(vqm_runtime *rt, const char *weight, const char *out);

/* set_gemm_min_rows(n) - qwen_runtime.cu:2324-2330: passes of n or more activation rows take the tensor-core GEMM
 * (fp16 operands, fp32 accumulation, like the reference's prompt kernel); 0 = never, every pass is fp32 matvecs. */
int vqm_set_gemm_min_rows(vqm_runtime *rt, int n);
/* synchronize() / mem_info() - qwen_runtime.cu:2267-2278.  synchronize also reports a kernel whose
 * bounded wait expired as VQM_ERR_CUDA. */
int vqm_synchronize(vqm_runtime *rt);
int vqm_mem_info(size_t *free_bytes, size_t *total_bytes);

/* The runtime's stream (a cudaStream_t), so that a caller can record events on it or order other work. */
void *vqm_stream(vqm_runtime *rt);
/* Makes the runtime launch on a stream the caller owns (for instance the stream another library is
 * capturing into a graph, or one that also carries NCCL collectives); NULL restores the runtime's own. */
int vqm_set_stream(vqm_runtime *rt, void *stream);
/* Records the launches made between begin and end into a CUDA graph instead of running them (a whole
 * decoder pass of qmv calls becomes one launch).  Blocking entry points are not allowed in between. */
int vqm_capture_begin(vqm_runtime *rt);
int vqm_capture_end(vqm_runtime *rt, int *graph_id);
int vqm_graph_launch(vqm_runtime *rt, int graph_id);
int vqm_graph_destroy(vqm_runtime *rt, int graph_id);
/* Number of kernels this runtime has launched (graph launches count their kernels). */
int vqm_launch_count(vqm_runtime *rt, uint64_t *out);

/* Stateless entry point for callers that own all memory: y = W x on `stream` (a cudaStream_t, NULL = legacy
 * default).  w: raw blocks, 16-byte aligned and readable 16 bytes past the end; x: [ntok][cols], y:
 * [ntok][rows], 16-byte aligned fp32; codebook: device copy of the type's codebook or NULL; status: device
 * word that receives a non-zero code if a bounded wait expires (may not be NULL).  1 <= ntok <= 8.
 * One device per process and one host thread at a time: the launch configuration of a kernel is cached per process, so
 * a call with another device current than the one this process launched on first returns VQM_ERR_VALUE (this holds for
 * vqm_runtime_create too). */
int vqm_qmv_raw(int type, const void *w, int rows, int cols, const float *x, float *y, int ntok, const void *codebook,
                unsigned *status, void *stream);

/* ---- Row-sharded tensors over several GPUs (no counterpart in the reference, which is a single-GPU engine) ----
 * Every rank (one process per GPU) holds a contiguous slice of the rows of each weight tensor.  vqm_qmv_push is
 * qmv on the local slice fused with its all-gather: the lane that holds an output stores it into the gathered
 * [ntok][rows_total] layout inside EVERY rank's exchange region (plain stores over NVLink), and the last block of the
 * launch to finish writes this rank's push count of the slot into the flag table of every region; a kernel that
 * consumes the gathered vector waits (bounded) until each rank's flag shows as many pushes of the slot as this rank
 * has made itself.
 *   vqm_exchange_create   allocates this rank's region (zeroed) and returns its 64-byte CUDA IPC handle
 *   vqm_exchange_open     maps a peer's region from its handle
 *   vqm_exchange_config   region addresses of all ranks (own included), this rank, and where inside a region the
 *                         flag table (unsigned flags[n_slots][8]) and this rank's own push counts (unsigned
 *                         pushes[n_slots]) live
 *   vqm_qmv_push          y = W_slice x on buffers x, y (y: [ntok][rows of the slice]); then, if slot >= 0, push y to
 *                         dst_off inside every region as rows [row_begin, row_begin + rows) of [ntok][rows_total] and
 *                         signal `slot`.  If wait_slot >= 0, x is only read after every rank has pushed wait_slot as
 *                         often as this rank has: the launch that produced x when it precedes this one in the pass,
 *                         or - for the first kernel of a pass, waiting on the slot of the pass's last kernel - the
 *                         previous pass, which makes sure no rank is still reading the vectors about to be rewritten.
 *                         with_argmax: also run the fused argmax (ids offset by the tensor's argmax row base).
 * All ranks must issue the same sequence of pushes.  A wait that expires sets the status word (reported by
 * vqm_synchronize) instead of hanging. */
int vqm_exchange_create(vqm_runtime *rt, size_t bytes, void *ipc_handle_out, uint64_t *addr);
int vqm_exchange_open(vqm_runtime *rt, const void *ipc_handle, uint64_t *addr);
int vqm_exchange_config(vqm_runtime *rt, int n_ranks, int rank, const uint64_t *region_addrs, size_t flag_off, size_t count_off,
                        int n_slots);
int vqm_qmv_push(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int slot, size_t dst_off, int rows_total,
                 int row_begin, int wait_slot, int with_argmax);

/* ---- Several tensors in one launch (no counterpart in the reference, which launches one kernel per tensor) ----
 * Tensors that read the same activations, share their GGUF type and have the same number of columns - the q/k/v
 * projections of an attention layer, the gate/up pair of an FFN - can be run by ONE launch: ys[i] = W_i x.  The
 * launch treats their rows as one list, so short tensors ride along with long ones instead of paying for a launch
 * each.  Every output equals, bit for bit, what vqm_qmv gives for its tensor alone, unless one of the two launches
 * is short enough to be split by columns (a launch whose rows would leave more than half of the GPU's warps idle
 * shares each row's columns among the up to 8 blocks of a thread-block cluster and adds their partial sums in column
 * order; the grouping of the additions then depends on the number of rows in the launch, never on ntok).
 *   n: 1..4 tensors; ntok: 1..8.  VQM_ERR_VALUE if the tensors do not share type and columns, or if a tensor's rows
 *   cannot follow the previous tensor's in one launch (for types whose rows are not multiples of 16 bytes, the row
 *   counts of all but the last tensor have to keep the rows' position within a 16-byte line going).
 * vqm_qmv_push_group is the row-sharded form (see vqm_qmv_push): per tensor its place in the gathered vectors, one
 * flag slot for the whole launch. */
int vqm_qmv_group(vqm_runtime *rt, int n, const char *const *weights, const char *x, const char *const *ys, int ntok);
/* Column split of short launches on (default) or off.  Off: every output is one warp's sum over all columns, so a
 * tensor's outputs do not depend on what else is in its launch; on: see above.  (The environment variable
 * VINF_B200_NO_SPLIT=1 sets the default to off.) */
int vqm_set_column_split(vqm_runtime *rt, int enabled);
int vqm_qmv_push_group(vqm_runtime *rt, int n, const char *const *weights, const char *x, const char *const *ys, int ntok, int slot,
                       const size_t *dst_offs, const int *rows_totals, const int *row_begins, int wait_slot);

/* No counterpart in the reference.  The LM-head matvec with fused argmax (like vqm_qmv_argmax) for callers that
 * must not allocate device memory - code inside a no-allocation region of a serving loop, a process whose GPU
 * memory was all handed out at start-up, a plugin limited to the buffers its host gave it.  Stateless: the caller
 * passes every input and output as a device pointer (w: raw blocks, 16-byte aligned, readable 16 bytes past the
 * end; x: [ntok][cols]; y: [ntok][rows] or NULL; out_ids: ntok ints; out_values: ntok floats or NULL; status: one
 * word that receives a non-zero code if a bounded wait expires), and the scratch the two phases of the argmax
 * share sits in a fixed 64.3 KB array inside the library (present on every GPU that loads the library until the
 * process exits).  It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Limits: 1 <= ntok <= 8 activation rows (more are refused with VQM_ERR_VALUE; split a wider pass into groups
 * of 8 yourself); the launch is capped at 1024 blocks, which is what the array has partial-result slots for.
 * The first call looks up the array's device address (cudaGetSymbolAddress, with the device current), and the first
 * call for each (type, ntok, shape class) configures its kernel (cudaFuncSetAttribute and an occupancy query, neither
 * of which allocates device memory): make one warm-up call per shape you will use before any stream capture and
 * before entering a region that forbids driver set-up work.  The caller zeroes *status before its first call; the
 * kernel only ever writes a non-zero code to it.  All calls share the one array, which keeps what the last call left in
 * it (the entry point re-zeroes the counter it needs); two calls that overlap on the GPU - different streams, or
 * different host threads - race on it and give undefined results.  Like vqm_qmv_raw it serves the one device this
 * process launched on first (VQM_ERR_VALUE with another device current). */
int vqm_qmv_argmax_static(int type, const void *w, int rows, int cols, const float *x, float *y, int ntok, const void *codebook,
                          int *out_ids, float *out_values, unsigned *status, void *stream);

/* No counterpart in the reference.  Measures, on the current device, how many scheduler cycles a warp instruction of the
 * kinds the matvec decoders are made of costs (one block per SM, warps_per_sm warps - a multiple of 4 in 4..32 - each
 * running 2048 x 16 independent instructions between two clock reads).  out[0..9]: PRMT, LOP3, FFMA2 (fma.rn.f32x2),
 * FFMA, IMAD, SHF, cvt.f32.f16, PRMT and FFMA2 alternating (per instruction), then the decode sequence of 8 packed 4-bit
 * weights of one row with 1 and with 4 activation rows (per 8 weights).  The instruction-issue roofline of the matvec
 * kernels is built on these numbers.  Allocates and frees a little device memory; synchronises the device. */
#define VQM_PROBE_KINDS 10
int vqm_probe_issue_rates(int warps_per_sm, double *out, int n);

#ifdef __cplusplus
}
#endif
#endif /* VINF_B200_H */
