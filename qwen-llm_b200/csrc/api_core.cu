// C ABI: library diagnostics, resident quantised matrices, the standalone few-row
// GEMM / argmax entry points and the two-GEMM "config 1" pipeline.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "gemm_ts.cuh"

namespace dfl {

static thread_local std::string t_last_error;
std::atomic<uint64_t> g_launches{0};
int sm_count() {
    static std::atomic<int> cached[16] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 16) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 16) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("DFL_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

void set_error(const std::string& msg) { t_last_error = msg; }
dfl_status fail(dfl_status st, const std::string& msg) {
    t_last_error = msg;
    return st;
}

// How a host thread waits for the device (stream and event synchronisation): the driver's default spins while there are
// fewer contexts than cores, which is the lowest latency for one driving thread and the wrong choice when many driving
// threads share the cores with the sampler's worker threads - a spinning waiter then takes a core from a thread that
// has work.  DFL_HOST_WAIT=block|yield|spin|auto (or dfl_set_host_wait) picks the policy per process.
namespace {
std::atomic<int> g_host_wait{-1};        // -1: environment not read yet; 0 auto, 1 spin, 2 yield, 3 block
std::atomic<uint32_t> g_wait_applied{0}; // bit d: device d carries the current policy
int host_wait_policy() {
    int p = g_host_wait.load(std::memory_order_acquire);
    if (p >= 0) return p;
    const char* e = std::getenv("DFL_HOST_WAIT");
    p = 0;
    if (e && !std::strcmp(e, "spin")) p = 1;
    else if (e && !std::strcmp(e, "yield")) p = 2;
    else if (e && !std::strcmp(e, "block")) p = 3;
    int expected = -1;
    g_host_wait.compare_exchange_strong(expected, p);
    return g_host_wait.load(std::memory_order_acquire);
}
}  // namespace

dfl_status use_device(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fail(DFL_ERR_NO_DEVICE, "no CUDA device is available; this library has no CPU path");
    }
    if (device < 0 || device >= n) return fail(DFL_ERR_BAD_ARG, "device index out of range");
    DFL_CUDA(cudaSetDevice(device));
    const int policy = host_wait_policy();
    if (policy > 0 && device < 32 && !(g_wait_applied.load(std::memory_order_acquire) & (1u << device))) {
        const unsigned flag = policy == 1 ? cudaDeviceScheduleSpin : policy == 2 ? cudaDeviceScheduleYield : cudaDeviceScheduleBlockingSync;
        DFL_CUDA(cudaSetDeviceFlags(flag));
        g_wait_applied.fetch_or(1u << device, std::memory_order_acq_rel);
    }
    return DFL_OK;
}

extern "C" dfl_status dfl_set_host_wait(int32_t mode) {
    if (mode < 0 || mode > 3) return fail(DFL_ERR_BAD_ARG, "set_host_wait: mode is 0 (driver default), 1 (spin), 2 (yield) or 3 (block)");
    g_host_wait.store(mode, std::memory_order_release);
    const uint32_t had = g_wait_applied.exchange(0, std::memory_order_acq_rel);   // every device takes the new policy at its next use
    if (mode == 0 && had) {   // back to the driver's default on the devices this library changed, and only on those
        int cur = 0;
        if (cudaGetDevice(&cur) == cudaSuccess) {
            for (int d = 0; d < 32; ++d)
                if ((had >> d & 1u) && cudaSetDevice(d) == cudaSuccess) cudaSetDeviceFlags(cudaDeviceScheduleAuto);
            cudaSetDevice(cur);
        }
        cudaGetLastError();
    }
    return DFL_OK;
}

// Reads the device error word; non-zero maps to a status.
dfl_status check_dev_err(cudaStream_t st, int* dev_err) {
    int h = 0;
    DFL_CUDA(cudaMemcpyAsync(&h, dev_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    DFL_CUDA(cudaStreamSynchronize(st));
    if (h == 0) return DFL_OK;
    int zero = 0;
    cudaMemcpyAsync(dev_err, &zero, sizeof(int), cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);
    switch (h) {
        case DEV_ERR_WAIT_FULL:
        case DEV_ERR_WAIT_EMPTY:
        case DEV_ERR_WAIT_DRAIN:
        case DEV_ERR_WAIT_PEER:
        case DEV_ERR_WAIT_FLAG: return fail(DFL_ERR_TIMEOUT, "device-side bounded wait gave up (code " + std::to_string(h) + ")");
        case DEV_ERR_OVERFLOW: return fail(DFL_ERR_CUDA, "activation outside the f16 operand range");
        case DEV_ERR_NONFINITE: return fail(DFL_ERR_ROUTE_STATUS, "expert routing met a NaN / Inf router logit (route status NONFINITE)");
        default: return fail(DFL_ERR_CUDA, "device error word " + std::to_string(h));
    }
}

dfl_status qmatrix_create(int device, int dtype, uint64_t n_in, uint64_t n_out, const void* data, uint64_t n_bytes,
                          bool on_device, cudaStream_t st, QMatrix* m, bool allow_ts, int kb_group) {
    DFL_CHECK(use_device(device));
    if (!data || n_in == 0 || n_out == 0) return fail(DFL_ERR_BAD_ARG, "qmatrix: null data or empty shape");
    m->device = device;
    m->dtype = dtype;
    m->n_in = n_in;
    m->n_out = n_out;
    if (dtype == DFL_F32) {
        if (n_bytes != n_in * n_out * 4) return fail(DFL_ERR_BAD_SHAPE, "qmatrix: f32 byte count mismatch");
        m->kblocks = 0;
        m->row_tiles = 0;
        DFL_CUDA(cudaMalloc(&m->tiles, n_bytes));
        DFL_CUDA(cudaMemcpyAsync(m->tiles, data, n_bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st));
        DFL_CUDA(cudaStreamSynchronize(st));
        return DFL_OK;
    }
    if (stage_bytes_of(dtype) == 0) return fail(DFL_ERR_UNSUPPORTED, "qmatrix: dtype " + std::to_string(dtype));
    if (n_in % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "qmatrix: n_in must be a multiple of 256");
    m->kblocks = (int)(n_in / TILE_K);
    m->row_tiles = (int)((n_out + TILE_R - 1) / TILE_R);
    if (n_bytes != m->ggml_bytes()) return fail(DFL_ERR_BAD_SHAPE, "qmatrix: byte count does not match dtype and shape");
    const uint8_t* src = static_cast<const uint8_t*>(data);
    uint8_t* tmp = nullptr;
    if (!on_device) {
        DFL_CUDA(cudaMalloc(&tmp, n_bytes));
        DFL_CUDA(cudaMemcpyAsync(tmp, data, n_bytes, cudaMemcpyHostToDevice, st));
        src = tmp;
    }
    m->layout = (allow_ts && ts_supported(dtype)) ? LAYOUT_TS : LAYOUT_FRAG;
    if (m->layout == LAYOUT_TS && dtype == DFL_Q8_0) {   // its scales are folded into the f16 operand: they have to leave room for q
        bool fits = false;
        const dfl_status fs = q80_scales_fit_ts(st, src, n_in, n_out, &fits);
        if (fs != DFL_OK) {
            if (tmp) cudaFree(tmp);
            return fs;
        }
        if (!fits) m->layout = LAYOUT_FRAG;
    }
    cudaError_t e = cudaMalloc(&m->tiles, m->bytes());   // the layout decides the resident size
    if (e != cudaSuccess) {
        if (tmp) cudaFree(tmp);
        return fail(DFL_ERR_OOM, std::string("qmatrix: cudaMalloc: ") + cudaGetErrorString(e));
    }
    if (kb_group > 0 && m->layout != LAYOUT_TS) {
        if (tmp) cudaFree(tmp);
        cudaFree(m->tiles);
        m->tiles = nullptr;
        return fail(DFL_ERR_UNSUPPORTED, "qmatrix: expert-grouped matrices need the tensor-memory GEMM (Q4_K / Q5_K / Q6_K / Q8_0 with scales in range)");
    }
    dfl_status s = m->layout == LAYOUT_TS ? retile_matrix_ts(st, dtype, src, n_in, n_out, m->tiles, kb_group)
                                          : retile_matrix(st, dtype, src, n_in, n_out, m->tiles);
    cudaError_t e2 = cudaStreamSynchronize(st);
    if (tmp) cudaFree(tmp);
    if (s != DFL_OK) return s;
    if (e2 != cudaSuccess) return fail(DFL_ERR_CUDA, std::string("qmatrix: retile: ") + cudaGetErrorString(e2));
    return DFL_OK;
}

void qmatrix_release(QMatrix* m) {
    if (m->tiles && m->owns) {
        cudaSetDevice(m->device);
        cudaFree(m->tiles);
    }
    m->tiles = nullptr;
}

}  // namespace dfl

using namespace dfl;

struct dfl_qmatrix {
    QMatrix m;
};

struct dfl_c1 {
    const dfl_qmatrix* w1;
    const dfl_qmatrix* head;
    cudaStream_t st;
    float *x, *part1, *h, *part2, *logits, *gap;
    uint8_t *acts1, *acts2;
    int32_t* argmax;
    void* am_scratch;
    int* err;
    int splits1, splits2;
    cudaEvent_t e0, e1;
    float* pinned;  // staging for results
};

extern "C" {

const char* dfl_version(void) { return "dflash_b200 0.1 (sm_100a)"; }
const char* dfl_last_error(void) { return t_last_error.c_str(); }
int32_t dfl_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
uint64_t dfl_launch_count(void) { return g_launches.load(); }

dfl_status dfl_qmatrix_create(int32_t device, int32_t dtype, uint64_t n_in, uint64_t n_out, const void* data, uint64_t n_bytes,
                              int32_t on_device, dfl_qmatrix** out) {
    if (!out) return fail(DFL_ERR_BAD_ARG, "qmatrix_create: out is null");
    *out = nullptr;
    auto* q = new dfl_qmatrix();
    dfl_status s = qmatrix_create(device, dtype, n_in, n_out, data, n_bytes, on_device != 0, 0, &q->m, true, 0);
    if (s != DFL_OK) {
        qmatrix_release(&q->m);
        delete q;
        return s;
    }
    *out = q;
    return DFL_OK;
}

void dfl_qmatrix_destroy(dfl_qmatrix* m) {
    if (!m) return;
    qmatrix_release(&m->m);
    delete m;
}

int32_t dfl_qmatrix_engine(const dfl_qmatrix* m) {
    if (!m || m->m.dtype == DFL_F32) return 0;
    return m->m.layout == LAYOUT_TS ? 2 : 1;
}

dfl_status dfl_qmatrix_dequant(const dfl_qmatrix* m, float* out_host, uint64_t n_floats) {
    if (!m || !out_host) return fail(DFL_ERR_BAD_ARG, "qmatrix_dequant: null argument");
    if (n_floats != m->m.n_in * m->m.n_out) return fail(DFL_ERR_BAD_SHAPE, "qmatrix_dequant: output size");
    DFL_CHECK(use_device(m->m.device));
    if (m->m.dtype == DFL_F32) {
        DFL_CUDA(cudaMemcpy(out_host, m->m.tiles, n_floats * 4, cudaMemcpyDeviceToHost));
        return DFL_OK;
    }
    float* d = nullptr;
    DFL_CUDA(cudaMalloc(&d, n_floats * 4));
    dfl_status s = m->m.layout == LAYOUT_TS ? decode_tiles_ts(0, m->m, d) : decode_tiles(0, m->m, d);
    cudaError_t e = cudaMemcpy(out_host, d, n_floats * 4, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (s != DFL_OK) return s;
    if (e != cudaSuccess) return fail(DFL_ERR_CUDA, cudaGetErrorString(e));
    return DFL_OK;
}

dfl_status dfl_fewrow_matmul(const dfl_qmatrix* m, const float* x_host, int32_t n_rows, float* y_host) {
    if (!m || !x_host || !y_host) return fail(DFL_ERR_BAD_ARG, "fewrow_matmul: null argument");
    if (n_rows < 1 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "fewrow_matmul: n_rows must be in [1, 16]");
    const QMatrix& q = m->m;
    if (q.dtype == DFL_F32) return fail(DFL_ERR_UNSUPPORTED, "fewrow_matmul: f32 matrices use the small-matrix kernel");
    DFL_CHECK(use_device(q.device));
    const int splits = gemm_choose_splits(q);
    float *x = nullptr, *part = nullptr, *y = nullptr;
    uint8_t* acts = nullptr;
    int* err = nullptr;
    dfl_status s = DFL_OK;
    auto cleanup = [&]() { cudaFree(x); cudaFree(part); cudaFree(y); cudaFree(acts); cudaFree(err); };
    if (cudaMalloc(&x, (size_t)n_rows * q.n_in * 4) != cudaSuccess || cudaMalloc(&part, (size_t)splits * MAX_ROWS * q.n_out * 4) != cudaSuccess ||
        cudaMalloc(&y, (size_t)n_rows * q.n_out * 4) != cudaSuccess || cudaMalloc(&acts, acts_bytes_for(q)) != cudaSuccess ||
        cudaMalloc(&err, 4) != cudaSuccess) {
        cleanup();
        return fail(DFL_ERR_OOM, "fewrow_matmul: cudaMalloc failed");
    }
    cudaMemset(err, 0, 4);
    cudaMemcpy(x, x_host, (size_t)n_rows * q.n_in * 4, cudaMemcpyHostToDevice);
    s = launch_prep_acts_for(0, q, x, (int)q.n_in, n_rows, 1.0f, acts, err);
    if (s == DFL_OK) s = launch_gemm_fewrow(0, q, acts, part, splits, GemmEpilogue{}, err, false);
    if (s == DFL_OK) s = launch_reduce_partials(0, part, splits, n_rows, q.n_out, y, (int)q.n_out);
    if (s == DFL_OK) s = check_dev_err(0, err);
    if (s == DFL_OK) {
        cudaError_t e = cudaMemcpy(y_host, y, (size_t)n_rows * q.n_out * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) s = fail(DFL_ERR_CUDA, cudaGetErrorString(e));
    }
    cleanup();
    return s;
}

dfl_status dfl_argmax_top2(int32_t device, const float* logits_host, int32_t n_rows, uint64_t vocab, int32_t* argmax_out,
                           float* gap_out) {
    if (!logits_host || !argmax_out || !gap_out) return fail(DFL_ERR_BAD_ARG, "argmax_top2: null argument");
    if (n_rows < 1 || n_rows > 1024 || vocab == 0) return fail(DFL_ERR_BAD_SHAPE, "argmax_top2: shape");
    DFL_CHECK(use_device(device));
    float *l = nullptr, *g = nullptr;
    int32_t* a = nullptr;
    void* sc = nullptr;
    auto cleanup = [&]() { cudaFree(l); cudaFree(g); cudaFree(a); cudaFree(sc); };
    if (cudaMalloc(&l, (size_t)n_rows * vocab * 4) != cudaSuccess || cudaMalloc(&g, n_rows * 4) != cudaSuccess ||
        cudaMalloc(&a, n_rows * 4) != cudaSuccess || cudaMalloc(&sc, (size_t)n_rows * ARGMAX_PARTS * 16) != cudaSuccess) {
        cleanup();
        return fail(DFL_ERR_OOM, "argmax_top2: cudaMalloc failed");
    }
    cudaMemcpy(l, logits_host, (size_t)n_rows * vocab * 4, cudaMemcpyHostToDevice);
    dfl_status s = launch_argmax_top2(0, l, n_rows, vocab, vocab, a, g, sc);
    if (s == DFL_OK) {
        cudaError_t e1 = cudaMemcpy(argmax_out, a, n_rows * 4, cudaMemcpyDeviceToHost);
        cudaError_t e2 = cudaMemcpy(gap_out, g, n_rows * 4, cudaMemcpyDeviceToHost);
        if (e1 != cudaSuccess || e2 != cudaSuccess) s = fail(DFL_ERR_CUDA, "argmax_top2: copy back failed");
    }
    cleanup();
    return s;
}

// ---- config 1 pipeline ---------------------------------------------------------
dfl_status dfl_c1_create(const dfl_qmatrix* w1, const dfl_qmatrix* head, dfl_c1** out) {
    if (!w1 || !head || !out) return fail(DFL_ERR_BAD_ARG, "c1_create: null argument");
    *out = nullptr;
    if (w1->m.n_out != head->m.n_in) return fail(DFL_ERR_BAD_SHAPE, "c1_create: head input width must equal W1 output width");
    if (w1->m.device != head->m.device) return fail(DFL_ERR_BAD_ARG, "c1_create: matrices on different devices");
    DFL_CHECK(use_device(w1->m.device));
    auto* p = new dfl_c1();
    p->w1 = w1;
    p->head = head;
    p->splits1 = gemm_choose_splits(w1->m);
    p->splits2 = gemm_choose_splits(head->m);
    const uint64_t k1 = w1->m.n_in, n1 = w1->m.n_out, v = head->m.n_out;
    bool ok = cudaStreamCreateWithFlags(&p->st, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMalloc(&p->x, MAX_ROWS * k1 * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->part1, (size_t)p->splits1 * MAX_ROWS * n1 * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->h, MAX_ROWS * n1 * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->part2, (size_t)p->splits2 * MAX_ROWS * v * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->logits, MAX_ROWS * v * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->gap, MAX_ROWS * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->argmax, MAX_ROWS * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&p->acts1, acts_bytes_for(w1->m)) == cudaSuccess;
    ok = ok && cudaMalloc(&p->acts2, acts_bytes_for(head->m)) == cudaSuccess;
    ok = ok && cudaMalloc(&p->am_scratch, MAX_ROWS * ARGMAX_PARTS * 16) == cudaSuccess;
    ok = ok && cudaMalloc(&p->err, 4) == cudaSuccess;
    ok = ok && cudaEventCreate(&p->e0) == cudaSuccess && cudaEventCreate(&p->e1) == cudaSuccess;
    ok = ok && cudaMallocHost(&p->pinned, MAX_ROWS * 8) == cudaSuccess;
    if (!ok) {
        dfl_c1_destroy(p);
        return fail(DFL_ERR_OOM, std::string("c1_create: allocation failed: ") + cudaGetErrorString(cudaGetLastError()));
    }
    cudaMemsetAsync(p->err, 0, 4, p->st);
    cudaStreamSynchronize(p->st);
    *out = p;
    return DFL_OK;
}

void dfl_c1_destroy(dfl_c1* p) {
    if (!p) return;
    cudaSetDevice(p->w1->m.device);
    cudaFree(p->x); cudaFree(p->part1); cudaFree(p->h); cudaFree(p->part2); cudaFree(p->logits); cudaFree(p->gap);
    cudaFree(p->argmax); cudaFree(p->acts1); cudaFree(p->acts2); cudaFree(p->am_scratch); cudaFree(p->err);
    if (p->pinned) cudaFreeHost(p->pinned);
    if (p->e0) cudaEventDestroy(p->e0);
    if (p->e1) cudaEventDestroy(p->e1);
    if (p->st) cudaStreamDestroy(p->st);
    delete p;
}

static dfl_status c1_enqueue(dfl_c1* p, int n_rows) {
    const QMatrix& a = p->w1->m;
    const QMatrix& b = p->head->m;
    DFL_CHECK(launch_prep_acts_for(p->st, a, p->x, (int)a.n_in, n_rows, 1.0f, p->acts1, p->err));
    DFL_CHECK(launch_gemm_fewrow(p->st, a, p->acts1, p->part1, p->splits1, GemmEpilogue{}, p->err, false));
    DFL_CHECK(launch_reduce_partials(p->st, p->part1, p->splits1, n_rows, a.n_out, p->h, (int)a.n_out));
    DFL_CHECK(launch_prep_acts_for(p->st, b, p->h, (int)a.n_out, n_rows, 1.0f, p->acts2, p->err));
    DFL_CHECK(launch_gemm_fewrow(p->st, b, p->acts2, p->part2, p->splits2, GemmEpilogue{}, p->err, false));
    DFL_CHECK(launch_reduce_partials(p->st, p->part2, p->splits2, n_rows, b.n_out, p->logits, (int)b.n_out));
    DFL_CHECK(launch_argmax_top2(p->st, p->logits, n_rows, b.n_out, b.n_out, p->argmax, p->gap, p->am_scratch));
    return DFL_OK;
}

dfl_status dfl_c1_upload(dfl_c1* p, const float* x_host, int32_t n_rows) {
    if (!p || !x_host) return fail(DFL_ERR_BAD_ARG, "c1_upload: null argument");
    if (n_rows < 1 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "c1: n_rows must be in [1, 16]");
    DFL_CHECK(use_device(p->w1->m.device));
    DFL_CUDA(cudaMemcpyAsync(p->x, x_host, (size_t)n_rows * p->w1->m.n_in * 4, cudaMemcpyHostToDevice, p->st));
    DFL_CUDA(cudaStreamSynchronize(p->st));
    return DFL_OK;
}

dfl_status dfl_c1_run_resident(dfl_c1* p, int32_t n_rows, int32_t iters, float* ms_total) {
    if (!p || !ms_total) return fail(DFL_ERR_BAD_ARG, "c1_run_resident: null argument");
    if (n_rows < 1 || n_rows > MAX_ROWS || iters < 1) return fail(DFL_ERR_BAD_SHAPE, "c1_run_resident: arguments");
    DFL_CHECK(use_device(p->w1->m.device));
    DFL_CUDA(cudaEventRecord(p->e0, p->st));
    for (int i = 0; i < iters; ++i) DFL_CHECK(c1_enqueue(p, n_rows));
    DFL_CUDA(cudaEventRecord(p->e1, p->st));
    DFL_CUDA(cudaEventSynchronize(p->e1));
    DFL_CUDA(cudaEventElapsedTime(ms_total, p->e0, p->e1));
    return check_dev_err(p->st, p->err);
}

dfl_status dfl_c1_step(dfl_c1* p, const float* x_host, int32_t n_rows, const int32_t* draft_ids, int32_t* argmax_out,
                       float* gap_out, int32_t* n_accepted, float* logits_host) {
    if (!p || !x_host || !argmax_out || !gap_out) return fail(DFL_ERR_BAD_ARG, "c1_step: null argument");
    if (n_rows < 1 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "c1: n_rows must be in [1, 16]");
    DFL_CHECK(use_device(p->w1->m.device));
    DFL_CUDA(cudaMemcpyAsync(p->x, x_host, (size_t)n_rows * p->w1->m.n_in * 4, cudaMemcpyHostToDevice, p->st));
    DFL_CHECK(c1_enqueue(p, n_rows));
    DFL_CUDA(cudaMemcpyAsync(p->pinned, p->argmax, n_rows * 4, cudaMemcpyDeviceToHost, p->st));
    DFL_CUDA(cudaMemcpyAsync(p->pinned + MAX_ROWS, p->gap, n_rows * 4, cudaMemcpyDeviceToHost, p->st));
    if (logits_host)
        DFL_CUDA(cudaMemcpyAsync(logits_host, p->logits, (size_t)n_rows * p->head->m.n_out * 4, cudaMemcpyDeviceToHost, p->st));
    DFL_CHECK(check_dev_err(p->st, p->err));  // synchronises the stream
    memcpy(argmax_out, p->pinned, n_rows * 4);
    memcpy(gap_out, p->pinned + MAX_ROWS, n_rows * 4);
    if (n_accepted && draft_ids) {
        // greedy prefix acceptance (crates/qwen-cli/src/qwen/dflash.rs:838-852)
        int n = 0;
        while (n < n_rows && draft_ids[n] == argmax_out[n]) ++n;
        *n_accepted = n;
    }
    return DFL_OK;
}

}  // extern "C"
