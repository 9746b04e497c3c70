// The runtime object behind the C ABI (include/vinf_b200.h): named weight tensors in raw GGUF block layout,
// named device buffers, and the entry points that launch the kernels.  Mirrors the quantized-matvec part of
// the reference's CPython type (engine/csrc/megakernel/qwen_runtime.cu:878-910 for the two records, :1198-1230
// for the lookups and their errors, :1338-1409 upload, :1616-1650 alloc, :1819-1912 write/read/qmv,
// :2167-2197 argmax, :2281-2315 matvec).  Weights are always resident: there is no host ring or VMM group.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <climits>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/vinf_b200.h"
#include "vqm_formats.cuh"
#include "vqm_kernels.h"

namespace {

thread_local std::string g_error = "";

int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
    return status;
}

int cuda_fail(const char *ctx, cudaError_t err) {
    // "<context> failed: <cudaGetErrorString>", the reference's message (qwen_runtime.cu:1100-1103)
    return fail(err == cudaErrorMemoryAllocation ? VQM_ERR_MEMORY : VQM_ERR_CUDA, "%s failed: %s", ctx, cudaGetErrorString(err));
}

struct Tensor {
    uint8_t *data = nullptr;
    int type = 0, rows = 0, cols = 0;
    size_t row_bytes = 0, nbytes = 0;
    int argmax_row_base = 0;
    bool owned = true;
};

struct Buffer {
    void *data = nullptr;
    size_t n = 0;
    int elem = 4;
    bool owned = true;
    size_t bytes() const { return n * static_cast<size_t>(elem); }
};

struct Graph {
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;
    bool uses_gemm_x = false;  // captured a prompt-pass GEMM, i.e. the address of the runtime's fp16 activation buffer
};

const char *const kCodebookNames[5] = {"iq2xxs_grid", "iq2xs_grid", "iq2s_grid", "iq3xxs_grid", "iq3s_grid"};
const int kCodebookTypes[5] = {vqm::kIQ2_XXS, vqm::kIQ2_XS, vqm::kIQ2_S, vqm::kIQ3_XXS, vqm::kIQ3_S};

}  // namespace

struct vqm_runtime {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;      // the stream in use
    cudaStream_t own_stream = nullptr;  // the one the runtime created
    std::unordered_map<std::string, Tensor> tensors;
    std::unordered_map<std::string, Buffer> buffers;
    uint8_t *codebooks[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    // fixed device scratch: status word, argmax partials/results
    unsigned *status = nullptr;
    unsigned *done_counter = nullptr;
    float *part_val = nullptr;
    int *part_idx = nullptr;
    int *argmax_ids = nullptr;     // [256]: fused argmax uses the first 8, argmax_rows up to 256
    float *argmax_vals = nullptr;  // [8]
    int allow_split = 1;  // short launches may be split by columns (VINF_B200_NO_SPLIT=1 turns it off)
    // scratch of the synchronous matvec entry
    float *scratch_x = nullptr, *scratch_y = nullptr;
    size_t scratch_x_n = 0, scratch_y_n = 0;
    void *gemm_x = nullptr;  // fp16 copy of the activations of a prompt pass
    size_t gemm_x_len = 0;   // in elements
    // exchange of row-sharded outputs between ranks
    void *exchange_own = nullptr;           // region this runtime allocated
    std::vector<void *> exchange_opened;    // peers' regions mapped through IPC handles
    vqm::PushInfo push{};                   // regions, rank, counters
    int exchange_slots = 0;
    int gemm_min_rows = 0;
    int gemm_tcgen05 = 1;    // prompt passes of 128+ rows run on the tcgen05 kernel (VINF_B200_GEMM=mma: warp-level MMA only)
    int overlap_launch = 1;  // programmatic dependent launch of consecutive matvecs (VINF_B200_NO_PDL=1 turns it off)
    bool capturing = false;
    uint64_t launches = 0, capture_launches = 0;
    bool capture_uses_gemm_x = false;
    std::vector<Graph> graphs;
    // file loader: per reader thread two pinned staging slots, a copy stream and an event per slot (created on first use)
    std::vector<uint8_t *> load_slots;
    std::vector<cudaStream_t> load_streams;
    std::vector<cudaEvent_t> load_events;
};

namespace {

const uint8_t *codebook_for(vqm_runtime *rt, int type) {
    for (int i = 0; i < 5; ++i)
        if (kCodebookTypes[i] == type) return rt->codebooks[i];
    return nullptr;
}

Tensor *find_tensor(vqm_runtime *rt, const char *name, int *status) {
    auto it = rt->tensors.find(name);
    if (it == rt->tensors.end()) {
        *status = fail(VQM_ERR_KEY, "weight tensor %s is not loaded", name);
        return nullptr;
    }
    return &it->second;
}

Buffer *find_any_buffer(vqm_runtime *rt, const char *name, int *status) {
    auto it = rt->buffers.find(name);
    if (it == rt->buffers.end()) {
        *status = fail(VQM_ERR_KEY, "device buffer %s is not allocated", name);
        return nullptr;
    }
    return &it->second;
}

// fp32 buffer with at least min_n elements (qwen_runtime.cu:1207-1222)
float *find_f32(vqm_runtime *rt, const char *name, size_t min_n, int *status) {
    Buffer *b = find_any_buffer(rt, name, status);
    if (b == nullptr) return nullptr;
    if (b->elem != 4) {
        *status = fail(VQM_ERR_TYPE, "device buffer %s is fp16 (KV cache), not fp32", name);
        return nullptr;
    }
    if (b->n < min_n) {
        *status = fail(VQM_ERR_VALUE, "device buffer %s has %zu floats, need %zu", name, b->n, min_n);
        return nullptr;
    }
    return static_cast<float *>(b->data);
}

void release(Tensor &t) {
    if (t.owned && t.data != nullptr) cudaFree(t.data);
    t.data = nullptr;
}
void release(Buffer &b) {
    if (b.owned && b.data != nullptr) cudaFree(b.data);
    b.data = nullptr;
}

// The launchers cache what they learn about a kernel (its shared-memory attribute, the blocks per SM) once per process, so
// every launch of a process has to go to the device the first one went to.  Returns VQM_OK or the error.
int check_one_device(int *dev_out, int *sm_count_out) {
    static int first_dev = -1, first_sm_count = 0;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail("cudaGetDevice", err);
    if (first_dev < 0) {
        err = cudaDeviceGetAttribute(&first_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return cuda_fail("device query", err);
        first_dev = dev;
    }
    if (dev != first_dev)
        return fail(VQM_ERR_VALUE, "this process has launched on device %d before; the library serves one device per process (current device: %d)",
                    first_dev, dev);
    if (dev_out != nullptr) *dev_out = dev;
    if (sm_count_out != nullptr) *sm_count_out = first_sm_count;
    return VQM_OK;
}

int no_capture(vqm_runtime *rt, const char *what) {
    if (rt->capturing) return fail(VQM_ERR_VALUE, "%s is not allowed while a graph is being captured", what);
    return VQM_OK;
}

void count_launch(vqm_runtime *rt, uint64_t n = 1) {
    if (rt->capturing) rt->capture_launches += n;
    else rt->launches += n;
}

cudaError_t dispatch_qmv(int type, const vqm::MatvecArgs &a, int m, int sm_count, cudaStream_t stream, int *grid) {
    switch (type) {
#define VQM_CASE(id, name) \
    case id: return a.fuse != 0 ? vqm::launch_qmv_fused_##name(a, m, sm_count, stream, grid) : vqm::launch_qmv_##name(a, m, sm_count, stream, grid);
        VQM_FOR_EACH_TYPE(VQM_CASE)
#undef VQM_CASE
        default: return cudaErrorInvalidValue;
    }
}

int check_shape(const char *name, int type, int cols, int rows, size_t *row_bytes) {
    const vqm::Traits t = vqm::traits_of(type);
    if (t.block == 0) return fail(VQM_ERR_VALUE, "unsupported GGUF tensor type id %d for CUDA matvec", type);
    if (cols <= 0 || rows <= 0 || cols % t.block != 0)
        return fail(VQM_ERR_VALUE, "%s: cols=%d must be a positive multiple of the block size", name, cols);
    *row_bytes = static_cast<size_t>(cols / t.block) * t.size;
    return VQM_OK;
}

void set_single_part(vqm::MatvecArgs &a, const uint8_t *w, float *y, int rows) {
    for (int i = 0; i < vqm::kMaxParts; ++i) a.part[i] = vqm::MatvecPart{nullptr, nullptr, INT_MAX, 0};
    a.part[0] = vqm::MatvecPart{w, y, rows, rows};
    a.rows = rows;
    a.k_split = 1;
}

// Launches y_p = W_p x for the n tensors of a group (same type and columns; one launch) and m <= 8 rows of x,
// optionally with the fused argmax (n = 1 only).
struct Fuse {
    int flags = 0;
    const float *x2 = nullptr, *norm_w = nullptr;
    float eps = 0.0f;
};

int launch_parts(vqm_runtime *rt, int n, const Tensor *const *ts, const float *x, float *const *ys, int m, bool with_argmax,
                 const vqm::PushInfo *push = nullptr, const Fuse *fuse = nullptr) {
    const Tensor &t0 = *ts[0];
    const uint8_t *cb = codebook_for(rt, t0.type);
    if (vqm::grid_is_codebook(t0.type) && cb == nullptr)
        return fail(VQM_ERR_VALUE, "the codebook for GGUF type %d has not been set (vqm_set_codebook)", t0.type);
    vqm::MatvecArgs a{};
    set_single_part(a, t0.data, ys[0], t0.rows);
    long long rows = t0.rows;
    for (int i = 1; i < n; ++i) {
        // the kernel derives where a row's bytes start inside its 16-byte line from the launch row number
        const uintptr_t want = (reinterpret_cast<uintptr_t>(t0.data) + static_cast<uintptr_t>(rows) * t0.row_bytes) & 15u;
        if ((reinterpret_cast<uintptr_t>(ts[i]->data) & 15u) != want)
            return fail(VQM_ERR_VALUE, "tensor %d of the group cannot follow the others in one launch (row alignment); launch it alone", i);
        rows += ts[i]->rows;
        if (rows > INT_MAX) return fail(VQM_ERR_VALUE, "too many rows in one launch");
        a.part[i] = vqm::MatvecPart{ts[i]->data, ys[i], static_cast<int>(rows), ts[i]->rows};
    }
    a.rows = static_cast<int>(rows);
    a.x = x;
    a.codebook = cb;
    a.status = rt->status;
    a.cols = t0.cols;
    a.row_bytes = static_cast<long long>(t0.row_bytes);
    a.overlap_launch = rt->overlap_launch;
    a.max_grid = vqm::kMaxGrid;
    a.allow_split = rt->allow_split;
    if (push != nullptr) {
        a.push = *push;
        a.done_counter = rt->done_counter;
    }
    if (fuse != nullptr) {
        a.fuse = fuse->flags;
        a.x2 = fuse->x2;
        a.norm_w = fuse->norm_w;
        a.eps = fuse->eps;
    }
    if (with_argmax) {
        a.part_val = rt->part_val;
        a.part_idx = rt->part_idx;
        a.done_counter = rt->done_counter;
        a.out_idx = rt->argmax_ids;
        a.out_val = rt->argmax_vals;
        a.row_base = t0.argmax_row_base;
    }
    const cudaError_t err = dispatch_qmv(t0.type, a, m, rt->sm_count, rt->stream, nullptr);
    if (err != cudaSuccess) return cuda_fail("qmv launch", err);
    count_launch(rt);
    return VQM_OK;
}

int launch_group(vqm_runtime *rt, const Tensor &t, const float *x, float *y, int m, bool with_argmax, const vqm::PushInfo *push = nullptr) {
    const Tensor *ts[1] = {&t};
    float *ys[1] = {y};
    return launch_parts(rt, 1, ts, x, ys, m, with_argmax, push);
}

// The tensors and output buffers of a group call, checked: same type and columns, every y large enough.
int resolve_group(vqm_runtime *rt, int n, const char *const *weights, const char *const *ys, int ntok, const Tensor **ts, float **yps) {
    if (n < 1 || n > vqm::kMaxParts) return fail(VQM_ERR_VALUE, "a group holds 1 to %d tensors", vqm::kMaxParts);
    if (weights == nullptr || ys == nullptr) return fail(VQM_ERR_VALUE, "null pointer");
    int rc = VQM_OK;
    for (int i = 0; i < n; ++i) {
        const Tensor *t = find_tensor(rt, weights[i], &rc);
        if (t == nullptr) return rc;
        if (t->cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weights[i]);
        if (i > 0 && (t->type != ts[0]->type || t->cols != ts[0]->cols))
            return fail(VQM_ERR_VALUE, "%s: the tensors of a group must share their GGUF type and their columns", weights[i]);
        ts[i] = t;
        yps[i] = find_f32(rt, ys[i], static_cast<size_t>(t->rows) * ntok, &rc);
        if (yps[i] == nullptr) return rc;
    }
    return VQM_OK;
}

int check_status_word(vqm_runtime *rt, const char *ctx) {
    unsigned host = 0;
    cudaError_t err = cudaMemcpyAsync(&host, rt->status, sizeof(host), cudaMemcpyDeviceToHost, rt->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail(ctx, err);
    if (host != 0) {
        cudaMemsetAsync(rt->status, 0, sizeof(unsigned), rt->stream);
        return fail(VQM_ERR_CUDA, "%s failed: a kernel gave up a bounded wait (status %u: 1 = its own weight copies, 2 = another rank's push)",
                    ctx, host);
    }
    return VQM_OK;
}

}  // namespace

extern "C" {

const char *vqm_last_error(void) { return g_error.c_str(); }

int vqm_runtime_create(const void *iq3s_grid, size_t nbytes, vqm_runtime **out) {
    if (out == nullptr) return fail(VQM_ERR_VALUE, "out must not be NULL");
    *out = nullptr;
    if (iq3s_grid != nullptr && nbytes != 2048)
        return fail(VQM_ERR_VALUE, "iq3s_grid must be 2048 bytes (512 entries x 4 values)");
    vqm_runtime *rt = new vqm_runtime();
    const int dev_rc = check_one_device(&rt->device, &rt->sm_count);
    if (dev_rc != VQM_OK) {
        delete rt;
        return dev_rc;
    }
    cudaError_t err = cudaSuccess;
    if (err == cudaSuccess) err = cudaStreamCreate(&rt->own_stream);
    rt->stream = rt->own_stream;
    if (err == cudaSuccess) err = cudaMalloc(&rt->status, 256);
    if (err == cudaSuccess) err = cudaMemset(rt->status, 0, 256);
    if (err == cudaSuccess) err = cudaMalloc(&rt->part_val, sizeof(float) * 8 * vqm::kMaxGrid);
    if (err == cudaSuccess) err = cudaMalloc(&rt->part_idx, sizeof(int) * 8 * vqm::kMaxGrid);
    if (err == cudaSuccess) err = cudaMalloc(&rt->argmax_ids, sizeof(int) * 256);
    if (err == cudaSuccess) err = cudaMalloc(&rt->argmax_vals, sizeof(float) * 8);
    if (err != cudaSuccess) {
        const int rc = cuda_fail("runtime setup", err);
        vqm_runtime_destroy(rt);
        return rc;
    }
    rt->done_counter = rt->status + 16;
    if (const char *e = getenv("VINF_B200_NO_PDL"); e != nullptr && e[0] == '1') rt->overlap_launch = 0;
    if (const char *e = getenv("VINF_B200_NO_SPLIT"); e != nullptr && e[0] == '1') rt->allow_split = 0;
    if (const char *e = getenv("VINF_B200_GEMM"); e != nullptr && strcmp(e, "mma") == 0) rt->gemm_tcgen05 = 0;
    if (iq3s_grid != nullptr) {
        const int rc = vqm_set_codebook(rt, "iq3s_grid", iq3s_grid, nbytes);
        if (rc != VQM_OK) {
            vqm_runtime_destroy(rt);
            return rc;
        }
    }
    *out = rt;
    return VQM_OK;
}

void vqm_runtime_destroy(vqm_runtime *rt) {
    if (rt == nullptr) return;
    if (rt->stream != nullptr) cudaStreamSynchronize(rt->stream);
    rt->stream = rt->own_stream;
    for (auto &g : rt->graphs)
        if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
    for (auto &kv : rt->tensors) release(kv.second);
    for (auto &kv : rt->buffers) release(kv.second);
    for (auto &cb : rt->codebooks) cudaFree(cb);
    cudaFree(rt->status);
    cudaFree(rt->part_val);
    cudaFree(rt->part_idx);
    cudaFree(rt->argmax_ids);
    cudaFree(rt->argmax_vals);
    cudaFree(rt->scratch_x);
    cudaFree(rt->scratch_y);
    cudaFree(rt->gemm_x);
    for (void *p : rt->exchange_opened) cudaIpcCloseMemHandle(p);
    cudaFree(rt->exchange_own);
    for (uint8_t *p : rt->load_slots) cudaFreeHost(p);
    for (cudaStream_t st : rt->load_streams) cudaStreamDestroy(st);
    for (cudaEvent_t ev : rt->load_events) cudaEventDestroy(ev);
    if (rt->stream != nullptr) cudaStreamDestroy(rt->stream);
    delete rt;
}

int vqm_set_codebook(vqm_runtime *rt, const char *name, const void *data, size_t nbytes) {
    for (int i = 0; i < 5; ++i) {
        if (strcmp(name, kCodebookNames[i]) != 0) continue;
        const size_t want = static_cast<size_t>(vqm::grid_bytes(kCodebookTypes[i]));
        if (data == nullptr || nbytes != want) return fail(VQM_ERR_VALUE, "%s must be %zu bytes", name, want);
        cudaError_t err = cudaSuccess;
        if (rt->codebooks[i] == nullptr) err = cudaMalloc(&rt->codebooks[i], want);
        if (err == cudaSuccess) err = cudaMemcpy(rt->codebooks[i], data, want, cudaMemcpyHostToDevice);
        if (err != cudaSuccess) return cuda_fail("codebook upload", err);
        return VQM_OK;
    }
    return fail(VQM_ERR_KEY, "unknown codebook %s", name);
}

int vqm_upload(vqm_runtime *rt, const char *name, const void *data, size_t nbytes, int type, int cols, int rows) {
    size_t row_bytes = 0;
    int rc = check_shape(name, type, cols, rows, &row_bytes);
    if (rc != VQM_OK) return rc;
    const size_t want = row_bytes * static_cast<size_t>(rows);
    if (nbytes != want) return fail(VQM_ERR_VALUE, "%s: got %zu bytes, expected %zu", name, nbytes, want);
    if ((rc = no_capture(rt, "upload")) != VQM_OK) return rc;
    auto it = rt->tensors.find(name);
    if (it != rt->tensors.end()) {
        cudaStreamSynchronize(rt->stream);
        release(it->second);
        rt->tensors.erase(it);
    }
    Tensor t;
    // +16: bulk copies are widened to 16-byte boundaries and may read up to 15 bytes past the end
    const size_t padded = (want + 16 + 255) / 256 * 256;
    cudaError_t err = cudaMalloc(&t.data, padded);
    if (err == cudaSuccess) err = cudaMemset(t.data + want, 0, padded - want);
    if (err == cudaSuccess) err = cudaMemcpy(t.data, data, want, cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        release(t);
        return cuda_fail("upload tensor", err);
    }
    t.type = type;
    t.rows = rows;
    t.cols = cols;
    t.row_bytes = row_bytes;
    t.nbytes = want;
    rt->tensors[name] = t;
    return VQM_OK;
}

// Weights straight from a file into HBM (replaces the reference's mmap + one blocking cudaMemcpy per tensor,
// engine/src/vinf/cuda/qwen_runtime.py:68-86 with engine/src/vinf/gguf/parser.py:153-159, and with it the residency
// planner: every tensor ends up resident).  `threads` readers take the tensor's 8 MiB chunks in turn; each owns two
// pinned staging slots and a copy stream, so the pread of one chunk overlaps the host-to-device copy of the previous
// one and the readers overlap one another.  Synchronous like vqm_upload: on return the bytes are in device memory.
constexpr size_t kLoadChunk = 8u << 20;
constexpr int kMaxLoadThreads = 16;

int vqm_upload_file(vqm_runtime *rt, const char *name, const char *path, uint64_t offset, uint64_t nbytes, int type, int cols, int rows,
                    int threads) {
    size_t row_bytes = 0;
    int rc = check_shape(name, type, cols, rows, &row_bytes);
    if (rc != VQM_OK) return rc;
    const size_t want = row_bytes * static_cast<size_t>(rows);
    if (nbytes != want) return fail(VQM_ERR_VALUE, "%s: got %llu bytes, expected %zu", name, static_cast<unsigned long long>(nbytes), want);
    if (path == nullptr) return fail(VQM_ERR_VALUE, "path must not be NULL");
    if ((rc = no_capture(rt, "upload_file")) != VQM_OK) return rc;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(VQM_ERR_VALUE, "%s: cannot open %s: %s", name, path, strerror(errno));
    const off_t file_size = lseek(fd, 0, SEEK_END);
    if (file_size < 0 || static_cast<uint64_t>(file_size) < offset + nbytes) {
        close(fd);
        return fail(VQM_ERR_VALUE, "%s: %s has %lld bytes, the tensor needs [%llu, %llu)", name, path, static_cast<long long>(file_size),
                    static_cast<unsigned long long>(offset), static_cast<unsigned long long>(offset + nbytes));
    }
    const size_t n_chunks = (want + kLoadChunk - 1) / kLoadChunk;
    int n_threads = threads <= 0 ? 4 : threads > kMaxLoadThreads ? kMaxLoadThreads : threads;
    if (static_cast<size_t>(n_threads) > n_chunks) n_threads = static_cast<int>(n_chunks);
    cudaError_t err = cudaSuccess;
    while (static_cast<int>(rt->load_streams.size()) < n_threads && err == cudaSuccess) {  // staging for one more reader
        uint8_t *slots[2] = {nullptr, nullptr};
        cudaEvent_t events[2] = {nullptr, nullptr};
        cudaStream_t st = nullptr;
        for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
            err = cudaHostAlloc(reinterpret_cast<void **>(&slots[i]), kLoadChunk, cudaHostAllocDefault);
            if (err == cudaSuccess) err = cudaEventCreateWithFlags(&events[i], cudaEventDisableTiming);
        }
        if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
        if (err != cudaSuccess) {
            for (int i = 0; i < 2; ++i) {
                if (slots[i] != nullptr) cudaFreeHost(slots[i]);
                if (events[i] != nullptr) cudaEventDestroy(events[i]);
            }
            break;
        }
        rt->load_slots.push_back(slots[0]);
        rt->load_slots.push_back(slots[1]);
        rt->load_events.push_back(events[0]);
        rt->load_events.push_back(events[1]);
        rt->load_streams.push_back(st);
    }
    if (err != cudaSuccess) {
        close(fd);
        return cuda_fail("file loader staging", err);
    }
    auto it = rt->tensors.find(name);
    if (it != rt->tensors.end()) {
        cudaStreamSynchronize(rt->stream);
        release(it->second);
        rt->tensors.erase(it);
    }
    Tensor t;
    const size_t padded = (want + 16 + 255) / 256 * 256;  // as in vqm_upload
    err = cudaMalloc(&t.data, padded);
    if (err == cudaSuccess) err = cudaMemset(t.data + want, 0, padded - want);
    if (err != cudaSuccess) {
        close(fd);
        release(t);
        return cuda_fail("upload_file", err);
    }
    std::atomic<int> first_error{0};  // 0 fine, 1 read error, 2 CUDA error
    std::string read_error;
    cudaError_t cuda_error = cudaSuccess;
    auto reader = [&](int tid) {
        if (cudaSetDevice(rt->device) != cudaSuccess) {
            first_error = 2;
            return;
        }
        uint8_t *const *slots = &rt->load_slots[2 * tid];
        cudaEvent_t *events = &rt->load_events[2 * tid];
        bool used[2] = {false, false};
        int turn = 0;
        for (size_t chunk = static_cast<size_t>(tid); chunk < n_chunks && first_error == 0; chunk += static_cast<size_t>(n_threads), turn ^= 1) {
            if (used[turn] && cudaEventSynchronize(events[turn]) != cudaSuccess) {  // the slot's previous copy has left it
                first_error = 2;
                return;
            }
            const size_t at = chunk * kLoadChunk, len = want - at < kLoadChunk ? want - at : kLoadChunk;
            size_t done = 0;
            while (done < len) {
                const ssize_t got = pread(fd, slots[turn] + done, len - done, static_cast<off_t>(offset + at + done));
                if (got <= 0) {
                    if (got < 0 && errno == EINTR) continue;
                    int expected = 0;
                    if (first_error.compare_exchange_strong(expected, 1)) read_error = got == 0 ? "unexpected end of file" : strerror(errno);
                    return;
                }
                done += static_cast<size_t>(got);
            }
            cudaError_t e = cudaMemcpyAsync(t.data + at, slots[turn], len, cudaMemcpyHostToDevice, rt->load_streams[tid]);
            if (e == cudaSuccess) e = cudaEventRecord(events[turn], rt->load_streams[tid]);
            if (e != cudaSuccess) {
                int expected = 0;
                if (first_error.compare_exchange_strong(expected, 2)) cuda_error = e;
                return;
            }
            used[turn] = true;
        }
    };
    std::vector<std::thread> workers;
    for (int tid = 1; tid < n_threads; ++tid) workers.emplace_back(reader, tid);
    reader(0);
    for (auto &w : workers) w.join();
    for (int tid = 0; tid < n_threads; ++tid) {
        const cudaError_t e = cudaStreamSynchronize(rt->load_streams[tid]);
        if (e != cudaSuccess && first_error == 0) {
            first_error = 2;
            cuda_error = e;
        }
    }
    close(fd);
    if (first_error != 0) {
        release(t);
        if (first_error == 1) return fail(VQM_ERR_VALUE, "%s: reading %s failed: %s", name, path, read_error.c_str());
        return cuda_fail("upload_file copy", cuda_error);
    }
    t.type = type;
    t.rows = rows;
    t.cols = cols;
    t.row_bytes = row_bytes;
    t.nbytes = want;
    rt->tensors[name] = t;
    return VQM_OK;
}

int vqm_bind_tensor(vqm_runtime *rt, const char *name, const void *device_ptr, int type, int cols, int rows) {
    size_t row_bytes = 0;
    const int rc = check_shape(name, type, cols, rows, &row_bytes);
    if (rc != VQM_OK) return rc;
    if (device_ptr == nullptr || (reinterpret_cast<uintptr_t>(device_ptr) & 15u) != 0)
        return fail(VQM_ERR_VALUE, "%s: device pointer must be 16-byte aligned", name);
    auto it = rt->tensors.find(name);
    if (it != rt->tensors.end()) {
        cudaStreamSynchronize(rt->stream);
        release(it->second);
        rt->tensors.erase(it);
    }
    Tensor t;
    t.data = const_cast<uint8_t *>(static_cast<const uint8_t *>(device_ptr));
    t.owned = false;
    t.type = type;
    t.rows = rows;
    t.cols = cols;
    t.row_bytes = row_bytes;
    t.nbytes = row_bytes * static_cast<size_t>(rows);
    rt->tensors[name] = t;
    return VQM_OK;
}

int vqm_free(vqm_runtime *rt, const char *name) {
    auto it = rt->tensors.find(name);
    if (it == rt->tensors.end()) return fail(VQM_ERR_KEY, "%s", name);
    cudaStreamSynchronize(rt->stream);
    release(it->second);
    rt->tensors.erase(it);
    return VQM_OK;
}

int vqm_has(vqm_runtime *rt, const char *name, int *out) {
    *out = rt->tensors.count(name) != 0;
    return VQM_OK;
}

int vqm_device_bytes(vqm_runtime *rt, size_t *out) {
    size_t total = 0;
    for (auto &kv : rt->tensors) total += kv.second.nbytes;
    *out = total;
    return VQM_OK;
}

int vqm_tensor_info(vqm_runtime *rt, const char *name, vqm_tensor_info_t *out) {
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, name, &rc);
    if (t == nullptr) return rc;
    out->addr = reinterpret_cast<uintptr_t>(t->data);
    out->type = t->type;
    out->rows = t->rows;
    out->cols = t->cols;
    out->row_bytes = static_cast<int64_t>(t->row_bytes);
    out->nbytes = static_cast<int64_t>(t->nbytes);
    out->resident = 1;
    return VQM_OK;
}

int vqm_alloc(vqm_runtime *rt, const char *name, size_t n, int elem) {
    if (n == 0 || n > (static_cast<size_t>(1) << 62)) return fail(VQM_ERR_VALUE, "buffer %s size must be positive", name);
    if (elem != 4 && elem != 2) return fail(VQM_ERR_VALUE, "element size must be 4 (fp32) or 2 (fp16)");
    const int rc = no_capture(rt, "alloc");
    if (rc != VQM_OK) return rc;
    auto it = rt->buffers.find(name);
    if (it != rt->buffers.end()) {
        cudaStreamSynchronize(rt->stream);
        release(it->second);
        rt->buffers.erase(it);
    }
    Buffer b;
    b.elem = elem;
    b.n = n;
    cudaError_t err = cudaMalloc(&b.data, b.bytes());
    if (err == cudaSuccess) err = cudaMemset(b.data, 0, b.bytes());
    if (err != cudaSuccess) {
        release(b);
        return cuda_fail("cudaMalloc buffer", err);
    }
    rt->buffers[name] = b;
    return VQM_OK;
}

int vqm_bind(vqm_runtime *rt, const char *name, void *device_ptr, size_t n, int elem) {
    if (n == 0) return fail(VQM_ERR_VALUE, "buffer %s size must be positive", name);
    if (elem != 4 && elem != 2) return fail(VQM_ERR_VALUE, "element size must be 4 (fp32) or 2 (fp16)");
    if (device_ptr == nullptr || (reinterpret_cast<uintptr_t>(device_ptr) & 15u) != 0)
        return fail(VQM_ERR_VALUE, "%s: device pointer must be 16-byte aligned", name);
    auto it = rt->buffers.find(name);
    if (it != rt->buffers.end()) {
        cudaStreamSynchronize(rt->stream);
        release(it->second);
        rt->buffers.erase(it);
    }
    Buffer b;
    b.data = device_ptr;
    b.n = n;
    b.elem = elem;
    b.owned = false;
    rt->buffers[name] = b;
    return VQM_OK;
}

int vqm_release(vqm_runtime *rt, const char *name) {
    auto it = rt->buffers.find(name);
    if (it == rt->buffers.end()) return fail(VQM_ERR_KEY, "device buffer %s is not allocated", name);
    cudaStreamSynchronize(rt->stream);
    release(it->second);
    rt->buffers.erase(it);
    return VQM_OK;
}

int vqm_write(vqm_runtime *rt, const char *name, const void *data, size_t nbytes, size_t offset) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    if (nbytes % b->elem != 0 || offset > b->n || nbytes / b->elem > b->n - offset)
        return fail(VQM_ERR_VALUE, "write to %s: bad offset/size for %d-byte elements", name, b->elem);
    if ((rc = no_capture(rt, "write")) != VQM_OK) return rc;
    cudaError_t err = cudaMemcpyAsync(static_cast<char *>(b->data) + offset * b->elem, data, nbytes, cudaMemcpyHostToDevice, rt->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail("buffer write", err);
    return VQM_OK;
}

int vqm_read(vqm_runtime *rt, const char *name, void *out, size_t n, size_t offset) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    if (offset > b->n) return fail(VQM_ERR_VALUE, "bad read offset");
    if (n > b->n - offset) return fail(VQM_ERR_VALUE, "read of %zu elements exceeds buffer %s", n, name);
    if ((rc = no_capture(rt, "read")) != VQM_OK) return rc;
    cudaError_t err = cudaMemcpyAsync(out, static_cast<char *>(b->data) + offset * b->elem, n * b->elem, cudaMemcpyDeviceToHost, rt->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail("buffer read", err);
    return VQM_OK;
}

int vqm_copy(vqm_runtime *rt, const char *dst, size_t dst_off, const char *src, size_t src_off, size_t n) {
    int rc = VQM_OK;
    Buffer *d = find_any_buffer(rt, dst, &rc);
    if (d == nullptr) return rc;
    Buffer *s = find_any_buffer(rt, src, &rc);
    if (s == nullptr) return rc;
    if (d->elem != s->elem) return fail(VQM_ERR_TYPE, "copy between buffers of different precision");
    if (dst_off > d->n || n > d->n - dst_off || src_off > s->n || n > s->n - src_off)
        return fail(VQM_ERR_VALUE, "copy out of bounds (%s <- %s)", dst, src);
    const size_t e = static_cast<size_t>(d->elem);
    const cudaError_t err = cudaMemcpyAsync(static_cast<char *>(d->data) + dst_off * e, static_cast<char *>(s->data) + src_off * e,
                                            n * e, cudaMemcpyDeviceToDevice, rt->stream);
    if (err != cudaSuccess) return cuda_fail("buffer copy", err);
    return VQM_OK;
}

int vqm_zero_range(vqm_runtime *rt, const char *name, size_t offset, size_t n) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    if (offset > b->n || n > b->n - offset) return fail(VQM_ERR_VALUE, "zero_range out of bounds");
    const cudaError_t err = cudaMemsetAsync(static_cast<char *>(b->data) + offset * b->elem, 0, n * b->elem, rt->stream);
    if (err != cudaSuccess) return cuda_fail("cudaMemset", err);
    return VQM_OK;
}

int vqm_zero(vqm_runtime *rt, const char *name) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    return vqm_zero_range(rt, name, 0, b->n);
}

int vqm_buffer_ptr(vqm_runtime *rt, const char *name, uint64_t *addr, size_t *n) {
    int rc = VQM_OK;
    float *p = find_f32(rt, name, 0, &rc);
    if (p == nullptr) return rc;
    *addr = reinterpret_cast<uintptr_t>(p);
    *n = rt->buffers[name].n;
    return VQM_OK;
}

int vqm_buffer_elem(vqm_runtime *rt, const char *name, int *elem) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    *elem = b->elem;
    return VQM_OK;
}

int vqm_buffer_len(vqm_runtime *rt, const char *name, size_t *n) {
    int rc = VQM_OK;
    Buffer *b = find_any_buffer(rt, name, &rc);
    if (b == nullptr) return rc;
    *n = b->n;
    return VQM_OK;
}

int vqm_buffer_bytes(vqm_runtime *rt, size_t *out) {
    size_t total = 0;
    for (auto &kv : rt->buffers) total += kv.second.bytes();
    *out = total;
    return VQM_OK;
}

int vqm_qmv(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok) {
    if (ntok < 1) return fail(VQM_ERR_VALUE, "ntok must be positive");
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    if (t->cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weight);
    const float *xp = find_f32(rt, x, static_cast<size_t>(t->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    float *yp = find_f32(rt, y, static_cast<size_t>(t->rows) * ntok, &rc);
    if (yp == nullptr) return rc;
    // Prompt mode (gemm_min_rows > 0, as in the reference's Runtime_qmv): passes of that many rows or more take the
    // tensor-core GEMM, the weight is decoded once per 256 activation rows.
    if (rt->gemm_min_rows > 0 && ntok >= rt->gemm_min_rows) {
        const uint8_t *cb = codebook_for(rt, t->type);
        if (vqm::grid_is_codebook(t->type) && cb == nullptr)
            return fail(VQM_ERR_VALUE, "the codebook for GGUF type %d has not been set (vqm_set_codebook)", t->type);
        // tcgen05 kernel (activation buffer padded to 512 rows) from 64 rows on, the warp-level MMA kernel below that
        const bool tc5 = rt->gemm_tcgen05 && ntok >= 64 && vqm::gemm_tc5_supports(t->cols);
        const int tile = tc5 ? vqm::gemm_tc5_token_tile() : vqm::gemm_token_tile();
        const size_t need = static_cast<size_t>((ntok + tile - 1) / tile * tile) * t->cols;
        cudaError_t err = cudaSuccess;
        if (need > rt->gemm_x_len) {
            if ((rc = no_capture(rt, "growing the prompt-pass activation buffer")) != VQM_OK) return rc;
            // a live graph that captured a prompt pass holds the old buffer's address: it must be destroyed first
            for (const Graph &g : rt->graphs)
                if (g.exec != nullptr && g.uses_gemm_x)
                    return fail(VQM_ERR_VALUE, "a captured graph uses the prompt-pass activation buffer, which a pass of %d rows would have to "
                                               "grow: destroy that graph first (or run the widest prompt pass once before capturing)", ntok);
            cudaStreamSynchronize(rt->stream);
            cudaFree(rt->gemm_x);
            rt->gemm_x = nullptr;
            rt->gemm_x_len = 0;
            err = cudaMalloc(&rt->gemm_x, need * 2);
            if (err != cudaSuccess) return cuda_fail("prompt-pass activation buffer", err);
            rt->gemm_x_len = need;
        }
        err = vqm::launch_f32_to_f16_rows(xp, rt->gemm_x, static_cast<long long>(ntok) * t->cols, static_cast<long long>(need), rt->stream);
        if (err == cudaSuccess) {
            if (tc5)
                err = vqm::launch_qgemm_tc5(t->type, t->data, rt->gemm_x, yp, t->rows, t->cols, static_cast<long long>(t->row_bytes), ntok, cb,
                                            rt->status, rt->stream);
            else
                err = vqm::launch_qgemm(t->type, t->data, rt->gemm_x, yp, t->rows, t->cols, static_cast<long long>(t->row_bytes), ntok, cb, rt->stream);
        }
        if (err != cudaSuccess) return cuda_fail("qmv gemm launch", err);
        if (rt->capturing) rt->capture_uses_gemm_x = true;
        count_launch(rt, 2);
        return VQM_OK;
    }
    // every group of 8 activation rows re-reads the weight (from L2 when it fits)
    for (int c = 0; c < ntok; c += 8) {
        const int m = ntok - c < 8 ? ntok - c : 8;
        rc = launch_group(rt, *t, xp + static_cast<size_t>(c) * t->cols, yp + static_cast<size_t>(c) * t->rows, m, false);
        if (rc != VQM_OK) return rc;
    }
    return VQM_OK;
}

int vqm_qmv_argmax(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int *out_ids) {
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8] for the fused argmax");
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    if (t->cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weight);
    const float *xp = find_f32(rt, x, static_cast<size_t>(t->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    float *yp = nullptr;
    if (y != nullptr) {
        yp = find_f32(rt, y, static_cast<size_t>(t->rows) * ntok, &rc);
        if (yp == nullptr) return rc;
    }
    if (out_ids != nullptr && (rc = no_capture(rt, "a blocking qmv_argmax")) != VQM_OK) return rc;
    if ((rc = launch_group(rt, *t, xp, yp, ntok, true)) != VQM_OK) return rc;
    if (out_ids != nullptr) {
        cudaError_t err = cudaMemcpyAsync(out_ids, rt->argmax_ids, sizeof(int) * ntok, cudaMemcpyDeviceToHost, rt->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
        if (err != cudaSuccess) return cuda_fail("qmv_argmax", err);
    }
    return VQM_OK;
}

int vqm_qmv_fused(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int flags, const char *x2, const char *norm_weight,
                  float eps, int *out_ids) {
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8] for the fused matvec");
    if ((flags & ~(VQM_FUSE_ADD | VQM_FUSE_NORM | VQM_FUSE_ARGMAX | VQM_FUSE_SILU_MUL)) != 0) return fail(VQM_ERR_VALUE, "unknown flag bits %d", flags);
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    if (t->cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weight);
    const float *xp = find_f32(rt, x, static_cast<size_t>(t->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    float *yp = nullptr;
    if (y != nullptr) {
        yp = find_f32(rt, y, static_cast<size_t>(t->rows) * ntok, &rc);
        if (yp == nullptr) return rc;
    }
    const bool with_argmax = (flags & VQM_FUSE_ARGMAX) != 0;
    if (yp == nullptr && (!with_argmax || (flags & VQM_FUSE_ADD))) return fail(VQM_ERR_VALUE, "y may only be NULL for an argmax without a residual");
    if (!with_argmax && out_ids != nullptr) return fail(VQM_ERR_VALUE, "out_ids without VQM_FUSE_ARGMAX");
    Fuse f;
    f.flags = flags & (VQM_FUSE_ADD | VQM_FUSE_NORM | VQM_FUSE_SILU_MUL);
    f.eps = eps;
    if (flags & VQM_FUSE_SILU_MUL) {
        if (x2 == nullptr) return fail(VQM_ERR_VALUE, "VQM_FUSE_SILU_MUL needs x2");
        f.x2 = find_f32(rt, x2, static_cast<size_t>(t->cols) * ntok, &rc);
        if (f.x2 == nullptr) return rc;
    }
    if (flags & VQM_FUSE_NORM) {
        if (norm_weight == nullptr) return fail(VQM_ERR_VALUE, "VQM_FUSE_NORM needs norm_weight");
        // the norm weights are an fp32 buffer of `cols` values, or an F32 tensor with `cols` elements (the reference keeps
        // them as a one-dimensional F32 weight tensor)
        auto wt = rt->tensors.find(norm_weight);
        if (wt != rt->tensors.end()) {
            if (wt->second.type != vqm::kF32 || static_cast<long long>(wt->second.rows) * wt->second.cols != t->cols)
                return fail(VQM_ERR_VALUE, "%s: norm weights must be F32 with %d elements", norm_weight, t->cols);
            f.norm_w = reinterpret_cast<const float *>(wt->second.data);
        } else {
            f.norm_w = find_f32(rt, norm_weight, static_cast<size_t>(t->cols), &rc);
            if (f.norm_w == nullptr) return rc;
        }
        if (!(eps >= 0.0f)) return fail(VQM_ERR_VALUE, "eps must be >= 0");
    }
    if (out_ids != nullptr && (rc = no_capture(rt, "a blocking fused argmax")) != VQM_OK) return rc;
    const Tensor *ts[1] = {t};
    float *ys[1] = {yp};
    if ((rc = launch_parts(rt, 1, ts, xp, ys, ntok, with_argmax, nullptr, &f)) != VQM_OK) return rc;
    if (out_ids != nullptr) {
        cudaError_t err = cudaMemcpyAsync(out_ids, rt->argmax_ids, sizeof(int) * ntok, cudaMemcpyDeviceToHost, rt->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
        if (err != cudaSuccess) return cuda_fail("qmv_fused", err);
    }
    return VQM_OK;
}

int vqm_argmax_result(vqm_runtime *rt, uint64_t *ids_addr, uint64_t *values_addr) {
    if (ids_addr != nullptr) *ids_addr = reinterpret_cast<uintptr_t>(rt->argmax_ids);
    if (values_addr != nullptr) *values_addr = reinterpret_cast<uintptr_t>(rt->argmax_vals);
    return VQM_OK;
}

int vqm_argmax_fetch(vqm_runtime *rt, int ntok, int *ids, float *values) {
    if (ntok < 1 || ntok > 8 || ids == nullptr) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8] and ids not NULL");
    const int rc = no_capture(rt, "argmax_fetch");
    if (rc != VQM_OK) return rc;
    cudaError_t err = cudaMemcpyAsync(ids, rt->argmax_ids, sizeof(int) * ntok, cudaMemcpyDeviceToHost, rt->stream);
    if (err == cudaSuccess && values != nullptr)
        err = cudaMemcpyAsync(values, rt->argmax_vals, sizeof(float) * ntok, cudaMemcpyDeviceToHost, rt->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail("argmax_fetch", err);
    return VQM_OK;
}

int vqm_set_argmax_row_base(vqm_runtime *rt, const char *weight, int row_base) {
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    if (row_base < 0) return fail(VQM_ERR_VALUE, "row_base must be >= 0");
    t->argmax_row_base = row_base;
    return VQM_OK;
}

int vqm_matvec(vqm_runtime *rt, const char *weight, const float *x_host, size_t x_bytes, float *y_host, size_t y_bytes) {
    auto it = rt->tensors.find(weight);
    if (it == rt->tensors.end()) return fail(VQM_ERR_KEY, "%s is not resident on the GPU", weight);
    const Tensor &t = it->second;
    if (x_bytes != static_cast<size_t>(t.cols) * sizeof(float))
        return fail(VQM_ERR_VALUE, "%s: x has %zu bytes, expected %d float32", weight, x_bytes, t.cols);
    if (y_bytes < static_cast<size_t>(t.rows) * sizeof(float))
        return fail(VQM_ERR_VALUE, "%s: y has room for %zu bytes, need %zu", weight, y_bytes, static_cast<size_t>(t.rows) * sizeof(float));
    if (t.cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weight);
    int rc = no_capture(rt, "matvec");
    if (rc != VQM_OK) return rc;
    cudaError_t err = cudaSuccess;
    if (rt->scratch_x_n < static_cast<size_t>(t.cols)) {
        cudaFree(rt->scratch_x);
        rt->scratch_x = nullptr;
        rt->scratch_x_n = 0;
        err = cudaMalloc(&rt->scratch_x, sizeof(float) * t.cols);
        if (err == cudaSuccess) rt->scratch_x_n = t.cols;
    }
    if (err == cudaSuccess && rt->scratch_y_n < static_cast<size_t>(t.rows)) {
        cudaFree(rt->scratch_y);
        rt->scratch_y = nullptr;
        rt->scratch_y_n = 0;
        err = cudaMalloc(&rt->scratch_y, sizeof(float) * t.rows);
        if (err == cudaSuccess) rt->scratch_y_n = t.rows;
    }
    if (err != cudaSuccess) return cuda_fail("scratch allocation", err);
    err = cudaMemcpyAsync(rt->scratch_x, x_host, x_bytes, cudaMemcpyHostToDevice, rt->stream);
    if (err != cudaSuccess) return cuda_fail("qmatvec H2D", err);
    if ((rc = launch_group(rt, t, rt->scratch_x, rt->scratch_y, 1, false)) != VQM_OK) return rc;
    err = cudaMemcpyAsync(y_host, rt->scratch_y, sizeof(float) * t.rows, cudaMemcpyDeviceToHost, rt->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail("qmatvec", err);
    return check_status_word(rt, "qmatvec");
}

int vqm_argmax_rows(vqm_runtime *rt, const char *x, int n, int ntok, int *out) {
    if (ntok < 1 || ntok > 256) return fail(VQM_ERR_VALUE, "ntok must be in [1, %d]", 256);
    if (n < 1) return fail(VQM_ERR_VALUE, "n must be positive");
    int rc = VQM_OK;
    const float *xp = find_f32(rt, x, static_cast<size_t>(n) * ntok, &rc);
    if (xp == nullptr) return rc;
    if ((rc = no_capture(rt, "argmax")) != VQM_OK) return rc;
    cudaError_t err = vqm::launch_argmax_rows(xp, n, ntok, rt->argmax_ids, rt->stream);
    if (err == cudaSuccess) {
        count_launch(rt);
        err = cudaMemcpyAsync(out, rt->argmax_ids, sizeof(int) * ntok, cudaMemcpyDeviceToHost, rt->stream);
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(rt->stream);
    if (err != cudaSuccess) return cuda_fail("argmax_rows", err);
    return VQM_OK;
}

int vqm_argmax(vqm_runtime *rt, const char *x, int n, int *out) { return vqm_argmax_rows(rt, x, n, 1, out); }

int vqm_dequantize(vqm_runtime *rt, const char *weight, const char *out) {
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    const size_t numel = static_cast<size_t>(t->rows) * t->cols;
    if (numel % 8 != 0) return fail(VQM_ERR_VALUE, "%s: element count must be a multiple of 8", weight);
    float *op = find_f32(rt, out, numel, &rc);
    if (op == nullptr) return rc;
    const uint8_t *cb = codebook_for(rt, t->type);
    if (vqm::grid_is_codebook(t->type) && cb == nullptr)
        return fail(VQM_ERR_VALUE, "the codebook for GGUF type %d has not been set (vqm_set_codebook)", t->type);
    const cudaError_t err = vqm::launch_dequant(t->type, t->data, op, static_cast<long long>(numel), cb, rt->stream);
    if (err != cudaSuccess) return cuda_fail("dequantize launch", err);
    count_launch(rt);
    return VQM_OK;
}

int vqm_set_gemm_min_rows(vqm_runtime *rt, int n) {
    if (n < 0) return fail(VQM_ERR_VALUE, "gemm_min_rows must be >= 0");
    rt->gemm_min_rows = n;
    return VQM_OK;
}

int vqm_synchronize(vqm_runtime *rt) {
    const int rc = no_capture(rt, "synchronize");
    if (rc != VQM_OK) return rc;
    const cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return cuda_fail("synchronize", err);
    return check_status_word(rt, "synchronize");
}

int vqm_mem_info(size_t *free_bytes, size_t *total_bytes) {
    const cudaError_t err = cudaMemGetInfo(free_bytes, total_bytes);
    if (err != cudaSuccess) return cuda_fail("cudaMemGetInfo", err);
    return VQM_OK;
}

void *vqm_stream(vqm_runtime *rt) { return rt->stream; }

int vqm_set_stream(vqm_runtime *rt, void *stream) {
    const int rc = no_capture(rt, "set_stream");
    if (rc != VQM_OK) return rc;
    rt->stream = stream != nullptr ? static_cast<cudaStream_t>(stream) : rt->own_stream;
    return VQM_OK;
}

int vqm_capture_begin(vqm_runtime *rt) {
    if (rt->capturing) return fail(VQM_ERR_VALUE, "a capture is already open");
    const cudaError_t err = cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal);
    if (err != cudaSuccess) return cuda_fail("cudaStreamBeginCapture", err);
    rt->capturing = true;
    rt->capture_launches = 0;
    rt->capture_uses_gemm_x = false;
    return VQM_OK;
}

int vqm_capture_end(vqm_runtime *rt, int *graph_id) {
    if (!rt->capturing) return fail(VQM_ERR_VALUE, "no capture is open");
    rt->capturing = false;
    cudaGraph_t graph = nullptr;
    cudaError_t err = cudaStreamEndCapture(rt->stream, &graph);
    if (err != cudaSuccess) return cuda_fail("cudaStreamEndCapture", err);
    Graph g;
    err = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (err != cudaSuccess) return cuda_fail("cudaGraphInstantiate", err);
    g.kernels = rt->capture_launches;
    g.uses_gemm_x = rt->capture_uses_gemm_x;
    rt->graphs.push_back(g);
    *graph_id = static_cast<int>(rt->graphs.size()) - 1;
    return VQM_OK;
}

int vqm_graph_launch(vqm_runtime *rt, int graph_id) {
    if (graph_id < 0 || graph_id >= static_cast<int>(rt->graphs.size()) || rt->graphs[graph_id].exec == nullptr)
        return fail(VQM_ERR_KEY, "unknown graph %d", graph_id);
    const cudaError_t err = cudaGraphLaunch(rt->graphs[graph_id].exec, rt->stream);
    if (err != cudaSuccess) return cuda_fail("cudaGraphLaunch", err);
    count_launch(rt, rt->graphs[graph_id].kernels);
    return VQM_OK;
}

int vqm_graph_destroy(vqm_runtime *rt, int graph_id) {
    if (graph_id < 0 || graph_id >= static_cast<int>(rt->graphs.size()) || rt->graphs[graph_id].exec == nullptr)
        return fail(VQM_ERR_KEY, "unknown graph %d", graph_id);
    cudaStreamSynchronize(rt->stream);
    cudaGraphExecDestroy(rt->graphs[graph_id].exec);
    rt->graphs[graph_id].exec = nullptr;
    return VQM_OK;
}

int vqm_launch_count(vqm_runtime *rt, uint64_t *out) {
    *out = rt->launches;
    return VQM_OK;
}

// ---- row-sharded tensors: exchange regions and the fused push -----------------------------------------------

int vqm_exchange_create(vqm_runtime *rt, size_t bytes, void *ipc_handle_out, uint64_t *addr) {
    if (bytes == 0 || ipc_handle_out == nullptr || addr == nullptr) return fail(VQM_ERR_VALUE, "bad exchange region arguments");
    if (rt->exchange_own != nullptr) return fail(VQM_ERR_VALUE, "this runtime already has an exchange region");
    const int rc = no_capture(rt, "exchange_create");
    if (rc != VQM_OK) return rc;
    cudaError_t err = cudaMalloc(&rt->exchange_own, bytes);
    if (err == cudaSuccess) err = cudaMemset(rt->exchange_own, 0, bytes);
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, rt->exchange_own);
    if (err != cudaSuccess) {
        cudaFree(rt->exchange_own);
        rt->exchange_own = nullptr;
        return cuda_fail("exchange region", err);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(ipc_handle_out, &h, sizeof(h));
    *addr = reinterpret_cast<uintptr_t>(rt->exchange_own);
    return VQM_OK;
}

int vqm_exchange_open(vqm_runtime *rt, const void *ipc_handle, uint64_t *addr) {
    if (ipc_handle == nullptr || addr == nullptr) return fail(VQM_ERR_VALUE, "bad exchange region arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    void *p = nullptr;
    const cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) return cuda_fail("cudaIpcOpenMemHandle", err);
    rt->exchange_opened.push_back(p);
    *addr = reinterpret_cast<uintptr_t>(p);
    return VQM_OK;
}

int vqm_exchange_config(vqm_runtime *rt, int n_ranks, int rank, const uint64_t *region_addrs, size_t flag_off, size_t count_off,
                        int n_slots) {
    if (n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks || region_addrs == nullptr || n_slots < 1)
        return fail(VQM_ERR_VALUE, "exchange_config: 1..8 ranks, 0 <= rank < ranks, at least one slot");
    if ((flag_off & 3u) != 0 || (count_off & 3u) != 0) return fail(VQM_ERR_VALUE, "flag and count offsets must be 4-byte aligned");
    vqm::PushInfo p{};
    for (int i = 0; i < n_ranks; ++i) {
        if (region_addrs[i] == 0 || (region_addrs[i] & 15u) != 0) return fail(VQM_ERR_VALUE, "region %d is not a 16-byte aligned address", i);
        p.region[i] = region_addrs[i];
    }
    p.n_ranks = n_ranks;
    p.rank = rank;
    p.flag_off = static_cast<long long>(flag_off);
    p.pushes = reinterpret_cast<unsigned *>(region_addrs[rank] + count_off);
    rt->push = p;
    rt->exchange_slots = n_slots;
    return VQM_OK;
}

int vqm_qmv_push(vqm_runtime *rt, const char *weight, const char *x, const char *y, int ntok, int slot, size_t dst_off, int rows_total,
                 int row_begin, int wait_slot, int with_argmax) {
    if (rt->push.n_ranks == 0) return fail(VQM_ERR_VALUE, "exchange_config has not been called");
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8]");
    if (slot < -1 || slot >= rt->exchange_slots || wait_slot < -1 || wait_slot >= rt->exchange_slots)
        return fail(VQM_ERR_VALUE, "slot out of range");
    int rc = VQM_OK;
    Tensor *t = find_tensor(rt, weight, &rc);
    if (t == nullptr) return rc;
    if (t->cols % 32 != 0) return fail(VQM_ERR_VALUE, "%s: matvec cols must be a multiple of 32", weight);
    if (rows_total < t->rows || row_begin < 0 || row_begin + t->rows > rows_total || (dst_off & 15u) != 0)
        return fail(VQM_ERR_VALUE, "%s: slice [%d, %d) does not fit %d rows, or dst_off is not 16-byte aligned", weight, row_begin,
                    row_begin + t->rows, rows_total);
    const float *xp = find_f32(rt, x, static_cast<size_t>(t->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    float *yp = find_f32(rt, y, static_cast<size_t>(t->rows) * ntok, &rc);
    if (yp == nullptr) return rc;
    vqm::PushInfo p = rt->push;
    p.dst_off[0] = static_cast<long long>(dst_off);
    p.rows_total[0] = rows_total;
    p.row_begin[0] = row_begin;
    p.push_slot = slot + 1;
    p.wait_slot = wait_slot + 1;
    return launch_group(rt, *t, xp, yp, ntok, with_argmax != 0, &p);
}

int vqm_set_column_split(vqm_runtime *rt, int enabled) {
    rt->allow_split = enabled != 0;
    return VQM_OK;
}

int vqm_qmv_group(vqm_runtime *rt, int n, const char *const *weights, const char *x, const char *const *ys, int ntok) {
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8]");
    const Tensor *ts[vqm::kMaxParts];
    float *yps[vqm::kMaxParts];
    int rc = resolve_group(rt, n, weights, ys, ntok, ts, yps);
    if (rc != VQM_OK) return rc;
    const float *xp = find_f32(rt, x, static_cast<size_t>(ts[0]->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    return launch_parts(rt, n, ts, xp, yps, ntok, false);
}

int vqm_qmv_push_group(vqm_runtime *rt, int n, const char *const *weights, const char *x, const char *const *ys, int ntok, int slot,
                       const size_t *dst_offs, const int *rows_totals, const int *row_begins, int wait_slot) {
    if (rt->push.n_ranks == 0) return fail(VQM_ERR_VALUE, "exchange_config has not been called");
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8]");
    if (slot < -1 || slot >= rt->exchange_slots || wait_slot < -1 || wait_slot >= rt->exchange_slots)
        return fail(VQM_ERR_VALUE, "slot out of range");
    if (dst_offs == nullptr || rows_totals == nullptr || row_begins == nullptr) return fail(VQM_ERR_VALUE, "null pointer");
    const Tensor *ts[vqm::kMaxParts];
    float *yps[vqm::kMaxParts];
    int rc = resolve_group(rt, n, weights, ys, ntok, ts, yps);
    if (rc != VQM_OK) return rc;
    const float *xp = find_f32(rt, x, static_cast<size_t>(ts[0]->cols) * ntok, &rc);
    if (xp == nullptr) return rc;
    vqm::PushInfo p = rt->push;
    for (int i = 0; i < n; ++i) {
        if (rows_totals[i] < ts[i]->rows || row_begins[i] < 0 || row_begins[i] + ts[i]->rows > rows_totals[i] || (dst_offs[i] & 15u) != 0)
            return fail(VQM_ERR_VALUE, "%s: slice [%d, %d) does not fit %d rows, or dst_off is not 16-byte aligned", weights[i], row_begins[i],
                        row_begins[i] + ts[i]->rows, rows_totals[i]);
        p.dst_off[i] = static_cast<long long>(dst_offs[i]);
        p.rows_total[i] = rows_totals[i];
        p.row_begin[i] = row_begins[i];
    }
    p.push_slot = slot + 1;
    p.wait_slot = wait_slot + 1;
    return launch_parts(rt, n, ts, xp, yps, ntok, false, &p);
}

int vqm_qmv_raw(int type, const void *w, int rows, int cols, const float *x, float *y, int ntok, const void *codebook,
                unsigned *status, void *stream) {
    size_t row_bytes = 0;
    const int rc = check_shape("w", type, cols, rows, &row_bytes);
    if (rc != VQM_OK) return rc;
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8]");
    if (cols % 32 != 0) return fail(VQM_ERR_VALUE, "matvec cols must be a multiple of 32");
    if (w == nullptr || x == nullptr || y == nullptr || status == nullptr) return fail(VQM_ERR_VALUE, "null pointer");
    if (((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) != 0)
        return fail(VQM_ERR_VALUE, "w, x and y must be 16-byte aligned");
    if (vqm::grid_is_codebook(type) && codebook == nullptr) return fail(VQM_ERR_VALUE, "GGUF type %d needs its codebook", type);
    int sm_count = 0;
    const int dev_rc = check_one_device(nullptr, &sm_count);
    if (dev_rc != VQM_OK) return dev_rc;
    vqm::MatvecArgs a{};
    set_single_part(a, static_cast<const uint8_t *>(w), y, rows);
    a.x = x;
    a.codebook = static_cast<const uint8_t *>(codebook);
    a.status = status;
    a.cols = cols;
    a.row_bytes = static_cast<long long>(row_bytes);
    const cudaError_t err = dispatch_qmv(type, a, ntok, sm_count, static_cast<cudaStream_t>(stream), nullptr);
    if (err != cudaSuccess) return cuda_fail("qmv launch", err);
    return VQM_OK;
}

// ---- fused matvec + argmax for callers that cannot allocate -------------------------------------------------
// The fused argmax needs a little device scratch between its two phases (per-block partial results and the
// "blocks done" counter).  vqm_qmv_argmax keeps that scratch in memory the runtime allocates when it is created.
// Some callers of this library are not able to do that: code running inside a region where the CUDA allocator
// must not be entered (a real-time serving loop with a no-allocation rule, a process whose memory was budgeted
// and handed out up front, a plugin that is only given the buffers its host decided on).  For them the scratch
// lives in this fixed array inside the library image; every GPU that loads the library carries these bytes until
// the process exits.
constexpr int kStaticMaxBlocks = 1024;  // largest grid the scratch below can serve
struct StaticArgmaxScratch {
    unsigned done_counter;
    unsigned pad[63];
    float part_val[8 * kStaticMaxBlocks];
    int part_idx[8 * kStaticMaxBlocks];
};
static __device__ __align__(256) unsigned char g_static_argmax_scratch[sizeof(StaticArgmaxScratch)];

int vqm_qmv_argmax_static(int type, const void *w, int rows, int cols, const float *x, float *y, int ntok, const void *codebook,
                          int *out_ids, float *out_values, unsigned *status, void *stream) {
    size_t row_bytes = 0;
    const int rc = check_shape("w", type, cols, rows, &row_bytes);
    if (rc != VQM_OK) return rc;
    if (ntok < 1 || ntok > 8) return fail(VQM_ERR_VALUE, "ntok must be in [1, 8]");
    if (cols % 32 != 0) return fail(VQM_ERR_VALUE, "matvec cols must be a multiple of 32");
    if (w == nullptr || x == nullptr || out_ids == nullptr || status == nullptr) return fail(VQM_ERR_VALUE, "null pointer");
    if (((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) != 0)
        return fail(VQM_ERR_VALUE, "w, x and y must be 16-byte aligned");
    if (vqm::grid_is_codebook(type) && codebook == nullptr) return fail(VQM_ERR_VALUE, "GGUF type %d needs its codebook", type);
    // Set-up, once per device and with that device current: the array's name is only a host-side handle, the kernel
    // needs the device address behind it.
    static StaticArgmaxScratch *scratch = nullptr;  // (one device per process, see check_one_device)
    int dev = 0, sm_count = 0;
    const int dev_rc = check_one_device(&dev, &sm_count);
    if (dev_rc != VQM_OK) return dev_rc;
    cudaError_t err = cudaSuccess;
    if (scratch == nullptr) {
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_static_argmax_scratch);
        if (err != cudaSuccess) return cuda_fail("cudaGetSymbolAddress", err);
        scratch = static_cast<StaticArgmaxScratch *>(ptr);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The counter must start at zero; an earlier call that was cut short could have left it otherwise.
    err = cudaMemsetAsync(&scratch->done_counter, 0, sizeof(unsigned), st);
    if (err != cudaSuccess) return cuda_fail("scratch reset", err);
    vqm::MatvecArgs a{};
    set_single_part(a, static_cast<const uint8_t *>(w), y, rows);
    a.x = x;
    a.codebook = static_cast<const uint8_t *>(codebook);
    a.status = status;
    a.part_val = scratch->part_val;
    a.part_idx = scratch->part_idx;
    a.done_counter = &scratch->done_counter;
    a.out_idx = out_ids;
    a.out_val = out_values;
    a.cols = cols;
    a.row_bytes = static_cast<long long>(row_bytes);
    a.max_grid = kStaticMaxBlocks;  // the launch never uses more blocks than the scratch has partial slots for
    int grid = 0;
    err = dispatch_qmv(type, a, ntok, sm_count, st, &grid);
    if (err != cudaSuccess) return cuda_fail("qmv launch", err);
    return VQM_OK;
}

}  // extern "C"
