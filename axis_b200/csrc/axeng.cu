// libaxeng.so — runtime and C ABI: buffer table, plan executor, CUDA-graph
// capture, NCCL data-parallel ops.  Kernels live in the other translation
// units of this directory; this file validates each op against the buffer
// table before anything is launched (an op that refers to a missing buffer or
// reaches past its end is refused with a code instead of faulting the GPU).
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include <cuda_runtime.h>
#include <nccl.h>

#include "../../include/axeng.h"
#include "kernels.h"

#define API extern "C" __attribute__((visibility("default")))
#define MAX_BUFS 65536
#define STAGE_SLOTS 4
#define RING_SLOTS 8
#define RING_FLOATS 64

struct Buf { void* p; long long bytes; bool owned; };

struct Engine {
    bool inited = false;
    cudaStream_t stream = nullptr, comm_stream = nullptr, side_stream = nullptr;    // main chain, collectives, overlapped weight-gradient GEMMs
    std::vector<cudaEvent_t> named_events;      // EVENT ops: cross-stream dependencies by id
    cudaStream_t cur = nullptr;                 // stream the next op goes to
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    std::vector<cudaEvent_t> fork_events;       // one per FORK/JOIN inside a plan
    size_t fork_used = 0;
    Buf bufs[MAX_BUFS];
    cudaGraphExec_t graph = nullptr;
    long long graph_launches = 0;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    int tf32 = 0, fallback = 0;
    int* d_status = nullptr;                    // device status word
    void* l2_flush = nullptr;                   // 256 MiB scratch written between timed repetitions
    long long bytes = 0, launches = 0;
    int profile = 0;
    float prof_ms[ENG_KIND_COUNT];
    int prof_calls[ENG_KIND_COUNT];
    int* stage[STAGE_SLOTS] = {nullptr};        // pinned token staging ring
    long long stage_cap[STAGE_SLOTS] = {0};
    cudaEvent_t stage_ev[STAGE_SLOTS] = {nullptr};
    int stage_next = 0;
    float* ring = nullptr;                      // pinned read-back ring: RING_SLOTS x RING_FLOATS
    cudaEvent_t ring_ev[RING_SLOTS] = {nullptr};
    int ring_ticket[RING_SLOTS];
    int ring_next = 0;
    char err[512] = {0};
    int last_op_rc = 0;
};
static Engine G;
int ax_variant = 0;

static void set_err(const char* fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(G.err, sizeof(G.err), fmt, ap);
    va_end(ap);
}

static void release_all() {
    if (G.stream) cudaStreamSynchronize(G.stream);
    if (G.comm_stream) cudaStreamSynchronize(G.comm_stream);
    if (G.side_stream) cudaStreamSynchronize(G.side_stream);
    if (G.graph) { cudaGraphExecDestroy(G.graph); G.graph = nullptr; }
    for (int i = 0; i < MAX_BUFS; i++) {
        if (G.bufs[i].p && G.bufs[i].owned) cudaFree(G.bufs[i].p);
        G.bufs[i].p = nullptr; G.bufs[i].bytes = 0; G.bufs[i].owned = false;
    }
    for (auto e : G.fork_events) cudaEventDestroy(e);
    G.fork_events.clear(); G.fork_used = 0;
    for (int i = 0; i < STAGE_SLOTS; i++) {
        if (G.stage[i]) cudaFreeHost(G.stage[i]);
        if (G.stage_ev[i]) cudaEventDestroy(G.stage_ev[i]);
        G.stage[i] = nullptr; G.stage_cap[i] = 0; G.stage_ev[i] = nullptr;
    }
    if (G.ring) { cudaFreeHost(G.ring); G.ring = nullptr; }
    for (int i = 0; i < RING_SLOTS; i++) {
        if (G.ring_ev[i]) cudaEventDestroy(G.ring_ev[i]);
        G.ring_ev[i] = nullptr; G.ring_ticket[i] = -1;
    }
    G.ring_next = 0;
    if (G.d_status) { cudaFree(G.d_status); G.d_status = nullptr; }
    if (G.l2_flush) { cudaFree(G.l2_flush); G.l2_flush = nullptr; }
    if (G.comm) { ncclCommDestroy(G.comm); G.comm = nullptr; }
    if (G.stream) { cudaStreamDestroy(G.stream); G.stream = nullptr; }
    if (G.comm_stream) { cudaStreamDestroy(G.comm_stream); G.comm_stream = nullptr; }
    if (G.side_stream) { cudaStreamDestroy(G.side_stream); G.side_stream = nullptr; }
    for (auto e : G.named_events) if (e) cudaEventDestroy(e);
    G.named_events.clear();
    G.bytes = 0; G.launches = 0; G.graph_launches = 0; G.inited = false;
}

API int eng_init(void) {
    if (G.inited) release_all();
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) { set_err("no CUDA device"); return 1; }
    // the main chain and the collectives get the highest priority, the side stream the lowest: its GEMMs take the
    // SMs the chain leaves idle and do not delay it (AXENG_FLAT_PRIORITY=1: all streams alike)
    int prio_lo = 0, prio_hi = 0;
    cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    if (getenv("AXENG_FLAT_PRIORITY")) prio_hi = prio_lo;
    if (cudaStreamCreateWithPriority(&G.stream, cudaStreamNonBlocking, prio_hi)) { set_err("stream create failed"); return 5; }
    if (cudaStreamCreateWithPriority(&G.comm_stream, cudaStreamNonBlocking, prio_hi)) { set_err("stream create failed"); return 5; }
    if (cudaStreamCreateWithPriority(&G.side_stream, cudaStreamNonBlocking, prio_lo)) { set_err("stream create failed"); return 5; }
    G.cur = G.stream;
    if (cudaMalloc(&G.d_status, 64)) { set_err("status alloc failed"); return 3; }
    cudaMemset(G.d_status, 0, 64);
    if (ax_gemm_tc_init()) { set_err("tensor-core GEMM init failed: %s", cudaGetErrorString(cudaGetLastError())); return 4; }
    if (ax_attn_tc_init()) { set_err("tensor-core attention init failed: %s", cudaGetErrorString(cudaGetLastError())); return 4; }
    memset(G.prof_ms, 0, sizeof(G.prof_ms));
    memset(G.prof_calls, 0, sizeof(G.prof_calls));
    G.inited = true; G.rank = 0; G.world = 1; G.fallback = 0;
    const char* fb = getenv("AXENG_FALLBACK");
    if (fb) G.fallback = atoi(fb);
    G.err[0] = 0;
    return 0;
}

API int eng_shutdown(void) { release_all(); return 0; }
API const char* eng_last_error(void) { return G.err; }
API int eng_has_flash(void) { return 1; }
API int eng_set_tf32(int on) { G.tf32 = on; return 0; }
API int eng_set_fallback(int mask) {
    G.fallback = mask;
    ax_gemm_set_mode((mask >> 2) & 3);      // 4: single-CTA GEMM only, 8: paired-CTA GEMM whenever possible
    return 0;
}
API long long eng_bytes_allocated(void) { return G.bytes; }
API int eng_last_variant(void) { return ax_variant; }
API int eng_sync(void) {
    int rc = (int)cudaStreamSynchronize(G.stream);
    if (!rc) rc = (int)cudaStreamSynchronize(G.comm_stream);
    if (!rc) rc = (int)cudaStreamSynchronize(G.side_stream);
    return rc;
}
API long long eng_launch_count(int reset) {
    long long v = G.launches;
    if (reset) G.launches = 0;
    return v;
}

static int alloc_common(int idx, long long nbytes, bool zero) {
    if (!G.inited) { set_err("engine not initialised"); return 1; }
    if (idx < 0 || idx >= MAX_BUFS) { set_err("buffer index %d out of range", idx); return 1; }
    if (nbytes < 0) { set_err("negative size"); return 1; }
    if (G.bufs[idx].p && G.bufs[idx].owned) { cudaFree(G.bufs[idx].p); G.bytes -= G.bufs[idx].bytes; }
    void* p = nullptr;
    const long long want = nbytes > 0 ? nbytes : 4;
    if (cudaMalloc(&p, (size_t)want) != cudaSuccess) {
        cudaGetLastError();
        set_err("cudaMalloc(%lld bytes) failed", want);
        return 2;
    }
    if (zero) cudaMemsetAsync(p, 0, (size_t)want, G.stream);
    G.bufs[idx].p = p; G.bufs[idx].bytes = want; G.bufs[idx].owned = true;
    G.bytes += want;
    return 0;
}
API int eng_alloc(int idx, long long nelems, int elsize) { return alloc_common(idx, nelems * elsize, false); }
API int eng_alloc_zero(int idx, long long nbytes) { return alloc_common(idx, nbytes, true); }
API int eng_alloc_view(int idx, int parent, long long byte_offset, long long nbytes) {
    if (idx < 0 || idx >= MAX_BUFS || parent < 0 || parent >= MAX_BUFS || !G.bufs[parent].p) { set_err("bad view"); return 1; }
    if (byte_offset < 0 || nbytes < 0 || byte_offset + nbytes > G.bufs[parent].bytes) { set_err("view exceeds parent"); return 1; }
    if (G.bufs[idx].p && G.bufs[idx].owned) { cudaFree(G.bufs[idx].p); G.bytes -= G.bufs[idx].bytes; }
    G.bufs[idx].p = (char*)G.bufs[parent].p + byte_offset;
    G.bufs[idx].bytes = nbytes; G.bufs[idx].owned = false;
    return 0;
}

static bool have(int idx, long long bytes_needed) {
    return idx >= 0 && idx < MAX_BUFS && G.bufs[idx].p && G.bufs[idx].bytes >= bytes_needed;
}

API int eng_upload(int idx, const float* host, long long nfloats) {
    if (!have(idx, nfloats * 4)) { set_err("upload: buffer %d missing or smaller than %lld floats", idx, nfloats); return 110; }
    return (int)cudaMemcpyAsync(G.bufs[idx].p, host, sizeof(float) * nfloats, cudaMemcpyHostToDevice, G.stream);
}
API int eng_download(int idx, float* host, long long nfloats) {
    if (!have(idx, nfloats * 4)) { set_err("download: buffer %d missing or smaller than %lld floats", idx, nfloats); return 110; }
    if (cudaMemcpyAsync(host, G.bufs[idx].p, sizeof(float) * nfloats, cudaMemcpyDeviceToHost, G.stream)) return 1;
    return (int)cudaStreamSynchronize(G.stream);
}
API int eng_upload_raw(int idx, long long off, const void* host, long long nbytes) {
    if (off < 0 || !have(idx, off + nbytes)) { set_err("upload_raw: out of range"); return 110; }
    return (int)cudaMemcpyAsync((char*)G.bufs[idx].p + off, host, nbytes, cudaMemcpyHostToDevice, G.stream);
}
API int eng_download_raw(int idx, long long off, void* host, long long nbytes) {
    if (off < 0 || !have(idx, off + nbytes)) { set_err("download_raw: out of range"); return 110; }
    if (cudaMemcpyAsync(host, (char*)G.bufs[idx].p + off, nbytes, cudaMemcpyDeviceToHost, G.stream)) return 1;
    return (int)cudaStreamSynchronize(G.stream);
}
// int64 host tokens -> int32 device ids through a pinned ring, so that the
// copy is truly asynchronous and the caller's array can be reused at once.
API int eng_upload_tokens(int idx, const long long* host, long long n, long long limit) {
    if (!have(idx, n * 4)) { set_err("upload_tokens: buffer %d too small", idx); return 110; }
    const int s = G.stage_next;
    G.stage_next = (s + 1) % STAGE_SLOTS;
    if (G.stage_cap[s] < n) {
        if (G.stage[s]) { cudaEventSynchronize(G.stage_ev[s]); cudaFreeHost(G.stage[s]); }
        if (cudaMallocHost(&G.stage[s], (size_t)n * 4)) { G.stage[s] = nullptr; G.stage_cap[s] = 0; set_err("pinned alloc failed"); return 2; }
        G.stage_cap[s] = n;
        if (!G.stage_ev[s]) cudaEventCreateWithFlags(&G.stage_ev[s], cudaEventDisableTiming);
    } else {
        cudaEventSynchronize(G.stage_ev[s]);
    }
    int* dst = G.stage[s];
    for (long long i = 0; i < n; i++) {
        const long long v = host[i];
        if (v >= limit || v < -1) { set_err("token %lld at %lld outside [-1, %lld)", v, i, limit); return 3; }
        dst[i] = (int)v;
    }
    int rc = (int)cudaMemcpyAsync(G.bufs[idx].p, dst, (size_t)n * 4, cudaMemcpyHostToDevice, G.stream);
    cudaEventRecord(G.stage_ev[s], G.stream);
    return rc;
}
API int eng_download_async(int idx, long long nfloats) {
    if (nfloats < 1 || nfloats > RING_FLOATS || !have(idx, nfloats * 4)) { set_err("download_async: buffer %d missing or count %lld outside 1..%d", idx, nfloats, RING_FLOATS); return -110; }
    if (!G.ring) {
        if (cudaMallocHost(&G.ring, sizeof(float) * RING_SLOTS * RING_FLOATS)) { G.ring = nullptr; set_err("pinned alloc failed"); return -2; }
        for (int i = 0; i < RING_SLOTS; i++) G.ring_ticket[i] = -1;
    }
    const int ticket = G.ring_next;
    const int s = ticket % RING_SLOTS;
    G.ring_next = ticket == 0x3fffffff ? 0 : ticket + 1;
    if (!G.ring_ev[s]) {
        if (cudaEventCreateWithFlags(&G.ring_ev[s], cudaEventDisableTiming)) { G.ring_ev[s] = nullptr; set_err("event create failed"); return -5; }
    } else if (G.ring_ticket[s] >= 0) {
        cudaEventSynchronize(G.ring_ev[s]);       // an uncollected copy into this slot: let it land before the slot is rewritten
    }
    if (cudaMemcpyAsync(G.ring + s * RING_FLOATS, G.bufs[idx].p, nfloats * 4, cudaMemcpyDeviceToHost, G.stream)) { set_err("download_async: copy failed"); return -1; }
    cudaEventRecord(G.ring_ev[s], G.stream);
    G.ring_ticket[s] = ticket;
    return ticket;
}
API int eng_download_wait(int ticket, float* host, long long nfloats) {
    const int s = ticket >= 0 ? ticket % RING_SLOTS : 0;
    if (ticket < 0 || !G.ring || G.ring_ticket[s] != ticket || nfloats < 1 || nfloats > RING_FLOATS) { set_err("download_wait: ticket %d is not pending", ticket); return 4; }
    if (cudaEventSynchronize(G.ring_ev[s])) { set_err("download_wait: %s", cudaGetErrorString(cudaGetLastError())); return 1; }
    memcpy(host, G.ring + s * RING_FLOATS, nfloats * 4);
    G.ring_ticket[s] = -1;
    return 0;
}
API int eng_device_status(int clear) {
    int v[16];
    cudaStreamSynchronize(G.stream);
    if (cudaMemcpy(v, G.d_status, 64, cudaMemcpyDeviceToHost)) return -1;
    if (clear) cudaMemset(G.d_status, 0, 64);
    return v[0];
}

// ── NCCL ────────────────────────────────────────────────────────────────────
API int eng_nccl_id(void* out128) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes");
    return (int)ncclGetUniqueId((ncclUniqueId*)out128);
}
API int eng_nccl_init_timeout(int rank, int world, const void* id128, int timeout_ms) {
    if (!G.inited) { set_err("engine not initialised"); return 1; }
    if (world < 1 || rank < 0 || rank >= world) { set_err("bad rank/world %d/%d", rank, world); return 8; }
    if (G.comm) { ncclCommDestroy(G.comm); G.comm = nullptr; }
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = ncclCommInitRankConfig(&G.comm, world, id, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) { set_err("ncclCommInitRankConfig: %s", ncclGetErrorString(r)); G.comm = nullptr; return (int)r; }
    const auto t0 = std::chrono::steady_clock::now();
    ncclResult_t st = ncclInProgress;
    while (true) {
        if (ncclCommGetAsyncError(G.comm, &st) != ncclSuccess) { st = ncclInternalError; break; }
        if (st != ncclInProgress) break;
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms > 0 && ms > timeout_ms) {
            ncclCommAbort(G.comm); G.comm = nullptr;
            set_err("nccl init timed out after %d ms (rank %d of %d)", timeout_ms, rank, world);
            return 7;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    if (st != ncclSuccess) { set_err("nccl init: %s", ncclGetErrorString(st)); ncclCommAbort(G.comm); G.comm = nullptr; return (int)st; }
    G.rank = rank; G.world = world;
    return 0;
}
API int eng_nccl_init(int rank, int world, const void* id128) {
    return eng_nccl_init_timeout(rank, world, id128, 0);
}
// non-blocking communicator: wait until an enqueue call has really been issued
static int nccl_wait(ncclResult_t r) {
    if (r == ncclSuccess) return 0;
    if (r != ncclInProgress) { set_err("nccl: %s", ncclGetErrorString(r)); return (int)r; }
    ncclResult_t st = ncclInProgress;
    const auto t0 = std::chrono::steady_clock::now();
    while (st == ncclInProgress) {
        if (ncclCommGetAsyncError(G.comm, &st) != ncclSuccess) return 9;
        if (std::chrono::duration_cast<std::chrono::seconds>(std::chrono::steady_clock::now() - t0).count() > 120) {
            set_err("nccl enqueue did not complete in 120 s");
            return 7;
        }
    }
    if (st != ncclSuccess) { set_err("nccl: %s", ncclGetErrorString(st)); return (int)st; }
    return 0;
}

// ── op execution ────────────────────────────────────────────────────────────
#define BUFP(i) (G.bufs[i].p)
#define NEED(idx, nbytes)                                                              \
    do {                                                                               \
        if (!have((idx), (long long)(nbytes))) {                                       \
            set_err("op kind %d: buffer %d missing or smaller than %lld bytes (has %lld)", op->kind, (idx), \
                    (long long)(nbytes), ((idx) >= 0 && (idx) < MAX_BUFS) ? G.bufs[idx].bytes : -1LL);       \
            return ((idx) < 0 || (idx) >= MAX_BUFS || !G.bufs[idx].p) ? 110 : 111;     \
        }                                                                              \
    } while (0)

static inline long long esz(int dt) { return dt == 1 ? 2 : 4; }

static int do_gemm(const EngOp* op, bool ex) {
    const int dt = op->dt;
    const bool in_bf = dt >= 1, out_bf = dt == 1;
    const long long ei = in_bf ? 2 : 4, eo = out_bf ? 2 : 4;
    const float alpha = op->alpha == 0.f ? 1.f : op->alpha;
    const float beta = op->beta;
    const int m = op->m, n = op->n, k = op->k;
    const int batch = op->batch > 0 ? op->batch : 1;
    if (m < 0 || n < 0 || k < 0 || op->tb < 0 || op->tb > 2) { set_err("gemm: bad shape"); return 112; }
    if (op->oa < 0 || op->ob < 0 || op->oc < 0 || (batch > 1 && (op->sa < 0 || op->sb < 0 || op->sc < 0))) {
        set_err("gemm: negative offset or batch stride"); return 112;
    }
    const long long a_el = (long long)m * k, b_el = (long long)k * n, c_el = (long long)m * n;
    NEED(op->a, (op->oa + (long long)(batch - 1) * op->sa + a_el) * ei);
    NEED(op->b, (op->ob + (long long)(batch - 1) * op->sb + b_el) * ei);
    NEED(op->c, (op->oc + (long long)(batch - 1) * op->sc + c_el) * eo);
    const char* A = (const char*)BUFP(op->a) + (long long)op->oa * ei;
    const char* B = (const char*)BUFP(op->b) + (long long)op->ob * ei;
    char* C = (char*)BUFP(op->c) + (long long)op->oc * eo;
    const char* D = C;
    if (ex && op->d >= 0) {
        NEED(op->d, (op->oc + (long long)(batch - 1) * op->sc + c_el) * eo);
        D = (const char*)BUFP(op->d) + (long long)op->oc * eo;
    }
    if (in_bf && batch == 1 && !(G.fallback & 1)) {
        const int rc = ax_gemm_tc(out_bf, op->tb, A, B, C, beta != 0.f ? D : nullptr, m, n, k, alpha, beta, G.d_status, G.cur);
        if (rc == 0) { G.launches++; return 0; }
        if (rc > 0) { set_err("tensor-core gemm failed rc=%d: %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
    }
    G.launches++;
    ax_variant = 0x20;
    return ax_gemm_simt(in_bf, out_bf, op->tb, A, B, C, beta != 0.f ? D : nullptr, m, n, k, batch,
                        op->sa, op->sb, op->sc, alpha, beta, G.cur);
}

// Several GEMMs of one layer as one launch.  tb/dt/alpha as GEMM; batch = count (2 or 3); oc = mode.
//   mode 1 (shared input): A = a; B_g = b, sa, sb; C_g = c, d, sc; n_g = n, oa, ob; k = k.
//   mode 2 (summed over K-segments): C = c; A_s = a, sa, sb; B_s = b, d, sc; k_s = k, oa, ob; n = n.
//   mode 3 (two independent problems of one depth k): A = a, sa; B = b, sb; C = c, d; m = m, oa; n = n, ob.
//   mode 4 (SwiGLU pair, batch = 2): A = a; gate weights b, up weights sa (both n wide); outputs g = c, u = d,
//           h = silu(g) * u = sc.
// When the grouped tensor-core kernel cannot serve the request (fp32 plan, shapes, alignment) the problems run
// one after another through the ordinary GEMM path: mode 2 as one GEMM plus accumulating ones.
// Extra operands announced by a GEMM_XSEG op for the next GEMM_GROUP op (host state of the single enqueueing thread).
//   a, b, d = A'_0..2   sa, sb, sc = B'_0..2 (0 / negative = none)   batch = how many   k = depth of each
//   c = addend buffer (mode 2 only, 0 / negative = none)   beta = its factor
// Before a mode-1 group: output g gets + A'_g B'_g.  Before a mode-2 group: the pairs are further K-segments of the sum
// (at most six in all) and the addend joins it: C = alpha * sum + beta * D.
static struct { int n, a[3], b[3], k, addend; float beta; } g_xseg = {};

static int do_gemm_xseg(const EngOp* op) {
    g_xseg = {};
    if (op->batch < 0 || op->batch > 3 || (op->batch > 0 && op->k < 1)) { set_err("gemm_xseg: bad count/depth"); return 112; }
    const int xa[3] = {op->a, op->b, op->d}, xb[3] = {op->sa, op->sb, op->sc};
    for (int g = 0; g < op->batch; g++) {
        if (xa[g] <= 0 || xb[g] <= 0) { set_err("gemm_xseg: operand %d missing", g); return 110; }
        g_xseg.a[g] = xa[g]; g_xseg.b[g] = xb[g];
    }
    g_xseg.n = op->batch; g_xseg.k = op->k;
    g_xseg.addend = op->c > 0 ? op->c : 0; g_xseg.beta = op->beta;
    if (g_xseg.n == 0 && !g_xseg.addend) { set_err("gemm_xseg: nothing to add"); return 112; }
    return 0;
}

// Adapter weight gradients out_g = alpha * X_g^T S_g of up to three projections (|batch| = count):
//   X_g = a, sa, sb (sa / sb <= 0: the same X as problem 0)   S_g = b, d, sc   F_g (columns of X_g) = n, k, tb
//   out_g = buffer c (fp32) at element offsets oa, ob, oc   m = tokens   gamma = rank R   beta = 1: out_g is [R, F_g]
//   (the transposed layout), else [F_g, R]   dt: 1 / 2 = bf16 inputs, 0 = fp32 inputs (GEMM path)
// batch < 0: the products are only noted (host state of the enqueueing thread, sixteen at most); batch == 0 runs all
// noted products as one launch — the adapters of a whole layer, whose operands are all still in place at the end of
// the layer's backward.  Tokens, rank and scale of a deferred set are those of its first op.
struct LoraGradItem { int x, s, c, off, F, layout; };
static struct { int n, N, R, dt; float alpha; LoraGradItem it[16]; } g_lgrad = {};

static int lora_grad_run(int count, const LoraGradItem* it, int N, int R, int dt, float alpha) {
    const void* X[16]; const void* S[16]; float* out[16]; int F[16], lay[16];
    for (int g = 0; g < count; g++) {
        X[g] = BUFP(it[g].x); S[g] = BUFP(it[g].s); out[g] = (float*)BUFP(it[g].c) + it[g].off;
        F[g] = it[g].F; lay[g] = it[g].layout;
    }
    if (dt >= 1 && !(G.fallback & 1)) {
        size_t wsb = 0;
        float* ws = ax_splitk_ws(&wsb);
        const int rc = ax_lora_grad(count, X, S, out, F, lay, N, R, alpha, ws, wsb, G.cur);
        if (rc == 0) { G.launches += 2; ax_variant = 0x60; return 0; }
        if (rc > 0) { set_err("lora_grad failed rc=%d: %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
    }
    for (int g = 0; g < count; g++) {          // as transposed-A GEMMs, one per product
        EngOp q = {};
        q.kind = ENG_GEMM_SB; q.batch = 1; q.tb = 2; q.dt = dt >= 1 ? 2 : 0; q.k = N; q.alpha = alpha; q.d = -1;
        q.c = it[g].c; q.oc = it[g].off;
        if (it[g].layout) { q.a = it[g].s; q.b = it[g].x; q.m = R; q.n = it[g].F; }
        else { q.a = it[g].x; q.b = it[g].s; q.m = it[g].F; q.n = R; }
        const int rc = do_gemm(&q, false);
        if (rc) return rc;
    }
    ax_variant = 0x61;
    return 0;
}

static int do_lora_grad(const EngOp* op) {
    if (op->batch == 0) {                      // run what was noted
        const auto p = g_lgrad;
        g_lgrad.n = 0;
        return p.n ? lora_grad_run(p.n, p.it, p.N, p.R, p.dt, p.alpha) : 0;
    }
    const bool defer = op->batch < 0;
    const int count = defer ? -op->batch : op->batch, R = (int)op->gamma, layout = op->beta != 0.f ? 1 : 0, N = op->m;
    if (count > 3 || R < 1 || N < 1) { set_err("lora_grad: bad count/rank/tokens"); return 112; }
    const int ix[3] = {op->a, op->sa > 0 ? op->sa : op->a, op->sb > 0 ? op->sb : op->a}, is[3] = {op->b, op->d, op->sc};
    const int F[3] = {op->n, op->k, op->tb}, off[3] = {op->oa, op->ob, op->oc};
    const long long ei = op->dt >= 1 ? 2 : 4;
    const float alpha = op->alpha == 0.f ? 1.f : op->alpha;
    LoraGradItem it[3];
    for (int g = 0; g < count; g++) {
        if (F[g] < 1 || off[g] < 0) { set_err("lora_grad: bad width/offset"); return 112; }
        NEED(ix[g], (long long)N * F[g] * ei); NEED(is[g], (long long)N * R * ei);
        NEED(op->c, ((long long)off[g] + (long long)F[g] * R) * 4);
        it[g] = {ix[g], is[g], op->c, off[g], F[g], layout};
    }
    if (!defer) return lora_grad_run(count, it, N, R, op->dt, alpha);
    if (g_lgrad.n == 0) { g_lgrad.N = N; g_lgrad.R = R; g_lgrad.dt = op->dt; g_lgrad.alpha = alpha; }
    if (g_lgrad.n + count > 16 || g_lgrad.N != N || g_lgrad.R != R || g_lgrad.dt != op->dt || g_lgrad.alpha != alpha) {
        g_lgrad.n = 0;
        set_err("lora_grad: a deferred set holds at most 16 products of one token count, rank, type and scale");
        return 112;
    }
    for (int g = 0; g < count; g++) g_lgrad.it[g_lgrad.n++] = it[g];
    return 0;
}

// The skinny products of adapters, out_g [m, R] = alpha * X_g W_g (batch = count <= 3):
//   X_g = a, sa, sb (sa / sb <= 0: the same X as problem 0) [m, F_g]   W_g = b, d, sc   out_g = buffers c, oa, ob
//   F_g = n, k, oc   tb = 0: W_g is [F_g, R] (u = x A), 1: [R, F_g] (t = g B^T)   gamma = R   dt as GEMM (0 / 1)
static int do_lora_proj(const EngOp* op) {
    const int count = op->batch, R = (int)op->gamma, N = op->m;
    if (count < 1 || count > 3 || R < 1 || N < 1 || op->tb < 0 || op->tb > 1) { set_err("lora_proj: bad count/rank/tokens/layout"); return 112; }
    const int ix[3] = {op->a, op->sa > 0 ? op->sa : op->a, op->sb > 0 ? op->sb : op->a}, iw[3] = {op->b, op->d, op->sc};
    const int io[3] = {op->c, op->oa, op->ob}, F[3] = {op->n, op->k, op->oc};
    const long long e = op->dt >= 1 ? 2 : 4;
    const float alpha = op->alpha == 0.f ? 1.f : op->alpha;
    const void* X[3]; const void* W[3]; void* out[3];
    for (int g = 0; g < count; g++) {
        if (F[g] < 1) { set_err("lora_proj: bad width"); return 112; }
        NEED(ix[g], (long long)N * F[g] * e); NEED(iw[g], (long long)F[g] * R * e); NEED(io[g], (long long)N * R * e);
        X[g] = BUFP(ix[g]); W[g] = BUFP(iw[g]); out[g] = BUFP(io[g]);
    }
    if (op->dt == 1 && !(G.fallback & 1)) {
        const int rc = ax_lora_proj(count, op->tb, X, W, out, F, N, R, alpha, G.cur);
        if (rc == 0) { G.launches++; ax_variant = 0x62; return 0; }
        if (rc > 0) { set_err("lora_proj failed rc=%d: %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
    }
    for (int g = 0; g < count; g++) {          // as GEMMs, one per product
        EngOp q = {};
        q.kind = ENG_GEMM_SB; q.batch = 1; q.tb = op->tb; q.dt = op->dt; q.alpha = alpha; q.d = -1;
        q.a = ix[g]; q.b = iw[g]; q.c = io[g]; q.m = N; q.n = R; q.k = F[g];
        const int rc = do_gemm(&q, false);
        if (rc) return rc;
    }
    ax_variant = 0x63;
    return 0;
}

static int do_gemm_group(const EngOp* op) {
    const int count = op->batch, mode = op->oc;
    const auto xs = g_xseg;                   // consumed by this op whatever happens
    g_xseg = {};
    if ((xs.n || xs.addend) && !(mode == 1 || mode == 2)) { set_err("gemm_group: extra operands need mode 1 or 2"); return 112; }
    if (mode == 1 && ((xs.n && xs.n != count) || xs.addend)) { set_err("gemm_group: mode 1 takes one extra term per output and no addend"); return 112; }
    if (count < (mode == 2 && xs.n ? 1 : 2) || count > 3 || mode < 1 || mode > 4 || ((mode == 3 || mode == 4) && count != 2)) { set_err("gemm_group: bad count/mode"); return 112; }
    if (mode == 4) {
        const int dt4 = op->dt;
        const long long e4 = dt4 == 1 ? 2 : 4;
        const long long mn = (long long)op->m * op->n;
        NEED(op->a, (long long)op->m * op->k * e4); NEED(op->b, (long long)op->k * op->n * e4); NEED(op->sa, (long long)op->k * op->n * e4);
        NEED(op->c, mn * e4); NEED(op->d, mn * e4); NEED(op->sc, mn * e4);
        if (dt4 == 1 && op->tb == 0 && !(G.fallback & 1) && !(G.fallback & 4)) {
            const void* A[1] = {BUFP(op->a)}; const void* B[2] = {BUFP(op->b), BUFP(op->sa)};
            void* C[3] = {BUFP(op->c), BUFP(op->d), BUFP(op->sc)};
            const float alpha = op->alpha == 0.f ? 1.f : op->alpha;
            const int rc = ax_gemm_tc2_group(1, 0, 4, 2, A, B, C, &op->m, &op->n, &op->k, alpha, G.d_status, G.cur);
            if (rc == 0) { G.launches++; return 0; }
            if (rc > 0) { set_err("fused SwiGLU gemm failed rc=%d: %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
        }
        // unfused: two GEMMs and the activation kernel
        EngOp g1 = *op; g1.kind = ENG_GEMM_SB; g1.batch = 1; g1.sa = g1.sb = g1.sc = 0; g1.oa = g1.ob = g1.oc = 0; g1.d = -1; g1.beta = 0.f;
        EngOp g2 = g1; g2.b = op->sa; g2.c = op->d;
        int rc = do_gemm(&g1, false);
        if (!rc) rc = do_gemm(&g2, false);
        if (rc) return rc;
        G.launches++;
        return ax_binary(2, dt4, BUFP(op->c), BUFP(op->d), BUFP(op->sc), mn, G.cur);
    }
    const int ia[3] = {op->a, op->sa, op->sb}, ib[3] = {op->b, mode == 1 ? op->sa : op->d, mode == 1 ? op->sb : op->sc};
    const int ic[3] = {op->c, op->d, op->sc}, dims[3] = {mode == 1 ? op->n : op->k, op->oa, op->ob};
    EngOp sub[6], xsub[3];
    int nsub = count;
    for (int g = 0; g < count; g++) {
        sub[g] = *op;
        sub[g].kind = ENG_GEMM_SB;
        sub[g].batch = 1; sub[g].sa = sub[g].sb = sub[g].sc = 0; sub[g].oa = sub[g].ob = sub[g].oc = 0; sub[g].d = -1;
        if (mode == 1) { sub[g].a = op->a; sub[g].b = ib[g]; sub[g].c = ic[g]; sub[g].n = dims[g]; sub[g].beta = 0.f; }
        else if (mode == 2) { sub[g].a = ia[g]; sub[g].b = ib[g]; sub[g].c = op->c; sub[g].k = dims[g]; sub[g].beta = g ? 1.f : 0.f; }
        else {
            sub[g].a = g ? op->sa : op->a; sub[g].b = g ? op->sb : op->b; sub[g].c = g ? op->d : op->c;
            sub[g].m = g ? op->oa : op->m; sub[g].n = g ? op->ob : op->n; sub[g].beta = 0.f;
        }
    }
    if (mode == 2) {
        for (int g = 0; g < xs.n; g++, nsub++) {            // further K-segments
            sub[nsub] = sub[0];
            sub[nsub].a = xs.a[g]; sub[nsub].b = xs.b[g]; sub[nsub].k = xs.k; sub[nsub].beta = 1.f;
        }
        if (xs.addend) { sub[0].kind = ENG_GEMM_EX; sub[0].d = xs.addend; sub[0].beta = xs.beta; }   // one-by-one form: the first product takes the addend
    } else if (mode == 1) {
        for (int g = 0; g < xs.n; g++) {                    // one-by-one form: C_g += A'_g B'_g
            xsub[g] = sub[g];
            xsub[g].a = xs.a[g]; xsub[g].b = xs.b[g]; xsub[g].k = xs.k; xsub[g].beta = 1.f;
        }
    }
    const int dt = op->dt;
    // mode 1 with gamma > 0: outputs 0 and 1 (the query and key projections) leave the op with the rotary embedding
    // applied; beta / gamma hold the buffer indices of the cos / sin tables ([T, 32] fp32: head_dim 64)
    const float* rcos = nullptr; const float* rsin = nullptr; int ropeT = 0;
    if (op->gamma > 0.f) {
        const int ic = (int)op->beta, is = (int)op->gamma;
        if (mode != 1 || count < 2 || op->tb != 0 || op->n % 64 || op->oa % 64) { set_err("gemm_group: rotary needs mode 1 and head_dim 64"); return 112; }
        NEED(ic, 128); NEED(is, 128);
        ropeT = (int)(G.bufs[ic].bytes / 128);
        NEED(is, (long long)ropeT * 128);
        rcos = (const float*)BUFP(ic); rsin = (const float*)BUFP(is);
    }
    if (dt >= 1 && !(G.fallback & 1) && !(G.fallback & 4)) {
        const long long ei = 2, eo = dt == 1 ? 2 : 4;
        const void* A[6]; const void* B[6]; void* C[6]; int mv[6], nv[6], kv[6];
        const void* XA[3] = {nullptr, nullptr, nullptr}; const void* XB[3] = {nullptr, nullptr, nullptr};
        for (int g = 0; g < nsub; g++) {
            const EngOp* q = &sub[g];
            NEED(q->a, (long long)q->m * q->k * ei); NEED(q->b, (long long)q->k * q->n * ei); NEED(q->c, (long long)q->m * q->n * eo);
            A[g] = BUFP(q->a); B[g] = BUFP(q->b); C[g] = BUFP(q->c); mv[g] = q->m; nv[g] = q->n; kv[g] = q->k;
        }
        if (mode == 1)
            for (int g = 0; g < xs.n; g++) {
                const EngOp* q = &xsub[g];
                NEED(q->a, (long long)q->m * q->k * ei); NEED(q->b, (long long)q->k * q->n * ei);
                XA[g] = BUFP(q->a); XB[g] = BUFP(q->b);
            }
        const void* D = nullptr;
        if (mode == 2 && xs.addend) { NEED(xs.addend, (long long)op->m * op->n * eo); D = BUFP(xs.addend); }
        const float alpha = op->alpha == 0.f ? 1.f : op->alpha;
        if (rcos) ax_gemm_group_rope(rcos, rsin, ropeT, 3);
        const int rc = ax_gemm_tc2_group(dt == 1, op->tb, mode, nsub, A, B, C, mv, nv, kv, alpha, G.d_status, G.cur,
                                         (mode == 1 && xs.n) ? XA : nullptr, XB, xs.k, D, xs.beta);
        if (rc == 0) { G.launches++; return 0; }
        if (rc > 0) { set_err("grouped tensor-core gemm failed rc=%d: %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
    }
    for (int g = 0; g < nsub; g++) {
        int rc = do_gemm(&sub[g], sub[g].kind == ENG_GEMM_EX);
        if (!rc && mode == 1 && g < xs.n) rc = do_gemm(&xsub[g], false);
        if (rc) return rc;
    }
    if (rcos) {          // unfused: the rotary kernel over the two projections, in place
        const long long e2 = esz(dt);
        NEED(op->c, (long long)op->m * op->n * e2); NEED(op->d, (long long)op->m * op->oa * e2);
        G.launches++;
        return ax_rope2(dt, BUFP(op->c), rcos, rsin, BUFP(op->c), ropeT, 64, (long long)op->m * (op->n / 64), op->n / 64, 0,
                        BUFP(op->d), BUFP(op->d), (long long)op->m * (op->oa / 64), op->oa / 64, G.cur);
    }
    return 0;
}

static AttnShape shape_bhtd(int B, int H, int KV, int T, int DH, float scale) {
    AttnShape s;
    s.B = B; s.H = H; s.KV = KV; s.T = T; s.DH = DH; s.scale = scale;
    s.qb = (long long)H * T * DH; s.qh = (long long)T * DH; s.qt = DH;
    s.kb = (long long)KV * T * DH; s.kh = (long long)T * DH; s.kt = DH;
    s.db = (long long)T * H; s.dh_ = 1; s.dtk = H;      // D laid out [B,T,H] (reference ROWDOT order)
    return s;
}
static AttnShape shape_bthd(int B, int H, int KV, int T, int DH, float scale) {
    AttnShape s;
    s.B = B; s.H = H; s.KV = KV; s.T = T; s.DH = DH; s.scale = scale;
    s.qb = (long long)T * H * DH; s.qh = DH; s.qt = (long long)H * DH;
    s.kb = (long long)T * KV * DH; s.kh = DH; s.kt = (long long)KV * DH;
    s.db = (long long)T * H; s.dh_ = 1; s.dtk = H;
    return s;
}

// rows of an embedding table (or of its gradient) that fit the buffer: ids are checked against it on the device
static int table_rows(int idx, int dim, long long elsize) {
    const long long r = dim > 0 ? G.bufs[idx].bytes / ((long long)dim * elsize) : 0;
    return r > 0x7fffffffLL ? 0x7fffffff : (int)r;
}

static int exec_op(const EngOp* op) {
    cudaStream_t st = G.cur;
    const int dt = op->dt;
    const long long es = esz(dt);
    switch (op->kind) {
        case ENG_GEMM: case ENG_GEMM_SB: return do_gemm(op, false);
        case ENG_GEMM_EX: return do_gemm(op, true);
        case ENG_GEMM_GROUP: return do_gemm_group(op);
        case ENG_GEMM_XSEG: return do_gemm_xseg(op);
        case ENG_LORA_GRAD: return do_lora_grad(op);
        case ENG_LORA_PROJ: return do_lora_proj(op);
        case ENG_ADD: case ENG_MUL: case ENG_SILU_MUL: {
            const long long n = op->n;
            NEED(op->a, n * es); NEED(op->b, n * es); NEED(op->c, n * es);
            G.launches++;
            return ax_binary(op->kind == ENG_ADD ? 0 : (op->kind == ENG_MUL ? 1 : 2), dt, BUFP(op->a), BUFP(op->b), BUFP(op->c), n, st);
        }
        case ENG_RMSNORM: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * es); NEED(op->b, op->n * es); NEED(op->c, el * es);
            G.launches++;
            return ax_rmsnorm(dt, BUFP(op->a), BUFP(op->b), BUFP(op->c), op->m, op->n, op->alpha, st);
        }
        case ENG_ADAMW: {
            const long long n = op->n;
            NEED(op->a, n * 4); NEED(op->b, n * 4); NEED(op->c, n * 4); NEED(op->d, n * 4);
            const float* tb = nullptr; void* pbf = nullptr; const float* lrb = nullptr; const float* gsb = nullptr;
            if (op->tb >= 0) { NEED(op->tb, 4); tb = (const float*)BUFP(op->tb); }
            if (op->sa > 0) { NEED(op->sa, n * 2); pbf = BUFP(op->sa); }
            if (op->sb > 0) { NEED(op->sb, 4); lrb = (const float*)BUFP(op->sb); }
            if (op->oa > 0) { NEED(op->oa, 4); gsb = (const float*)BUFP(op->oa); }
            G.launches++;
            return ax_adamw((float*)BUFP(op->a), (const float*)BUFP(op->b), (float*)BUFP(op->c), (float*)BUFP(op->d),
                            tb, pbf, lrb, gsb, op->alpha, op->beta, op->gamma, n, st);
        }
        case ENG_SCALE: {
            const long long n = op->n;
            NEED(op->c, n * es);
            if (op->alpha != 0.f) NEED(op->a, n * es);
            G.launches++;
            return ax_scale(dt, op->a >= 0 ? BUFP(op->a) : nullptr, BUFP(op->c), op->alpha, n, st);
        }
        case ENG_COPY: {
            const long long n = op->n;
            NEED(op->a, n * es); NEED(op->c, n * es);
            G.launches++;
            return ax_copy(dt, BUFP(op->a), BUFP(op->c), n, st);
        }
        case ENG_PERM_0213: {
            const long long el = (long long)op->m * op->n * op->k * op->batch;
            NEED(op->a, el * es); NEED(op->c, el * es);
            G.launches++;
            return ax_perm0213(dt, BUFP(op->a), BUFP(op->c), op->m, op->n, op->k, op->batch, st);
        }
        case ENG_ROPE: {
            const long long rows = (long long)op->batch * op->m;
            NEED(op->a, rows * op->n * es); NEED(op->c, rows * op->n * es);
            NEED(op->b, (long long)op->m * (op->n / 2) * 4); NEED(op->d, (long long)op->m * (op->n / 2) * 4);
            G.launches++;
            return ax_rope(dt, BUFP(op->a), (const float*)BUFP(op->b), (const float*)BUFP(op->d), BUFP(op->c), op->m, op->n, rows, 1, op->tb != 0, st);
        }
        case ENG_ROPE_BTHD: {
            // a=x b=cos d=sin c=out; batch=B m=T k=heads n=DH; tb=1 inverse; optional second tensor in the same
            // launch: sa=x2 sb=out2 sc=its heads (0 = none)
            const long long rows = (long long)op->batch * op->m * op->k;
            NEED(op->a, rows * op->n * es); NEED(op->c, rows * op->n * es);
            NEED(op->b, (long long)op->m * (op->n / 2) * 4); NEED(op->d, (long long)op->m * (op->n / 2) * 4);
            const void* x2 = nullptr; void* o2 = nullptr; long long rows2 = 0;
            if (op->sc > 0) {
                rows2 = (long long)op->batch * op->m * op->sc;
                NEED(op->sa, rows2 * op->n * es); NEED(op->sb, rows2 * op->n * es);
                x2 = BUFP(op->sa); o2 = BUFP(op->sb);
            }
            G.launches++;
            return ax_rope2(dt, BUFP(op->a), (const float*)BUFP(op->b), (const float*)BUFP(op->d), BUFP(op->c), op->m, op->n, rows, op->k,
                            op->tb != 0, x2, o2, rows2, op->sc, st);
        }
        case ENG_SOFTMAX_CAUSAL: {
            const long long rows = (long long)op->batch * op->m;
            const int width = op->n > 0 ? op->n : op->m;
            NEED(op->a, rows * width * es); NEED(op->c, rows * width * es);
            G.launches++;
            return ax_softmax_causal(dt, BUFP(op->a), BUFP(op->c), op->m, width, op->k, rows, st);
        }
        case ENG_SOFTMAX_BWD: {
            const long long rows = (long long)op->batch * op->m;
            const int width = op->n > 0 ? op->n : op->m;
            NEED(op->a, rows * width * es); NEED(op->b, rows * width * es); NEED(op->c, rows * width * es);
            G.launches++;
            return ax_softmax_bwd(dt, BUFP(op->a), BUFP(op->b), BUFP(op->c), width, rows, st);
        }
        case ENG_REPEAT_KV: case ENG_REPEAT_KV_BWD: {
            // batch=B, tb=KV, n=H, m=T, k=dh
            const long long big = (long long)op->batch * op->n * op->m * op->k, small = (long long)op->batch * op->tb * op->m * op->k;
            if (op->tb <= 0 || op->n % op->tb) { set_err("repeat_kv: H %% KV != 0"); return 112; }
            G.launches++;
            if (op->kind == ENG_REPEAT_KV) {
                NEED(op->a, small * es); NEED(op->c, big * es);
                return ax_repeat_kv(dt, BUFP(op->a), BUFP(op->c), op->batch, op->tb, op->n, op->m, op->k, st);
            }
            NEED(op->a, big * es); NEED(op->c, small * es);
            return ax_repeat_kv_bwd(dt, BUFP(op->a), BUFP(op->c), op->batch, op->tb, op->n, op->m, op->k, st);
        }
        case ENG_RMSNORM_BWD: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * es); NEED(op->b, op->n * es); NEED(op->d, el * es); NEED(op->c, el * es); NEED(op->tb, el * es);
            G.launches++;
            return ax_rmsnorm_bwd(dt, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), BUFP(op->tb), op->m, op->n, op->alpha, st);
        }
        case ENG_COLSUM: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * (dt >= 1 ? 2 : 4)); NEED(op->c, (long long)op->n * 4);
            G.launches++;
            return ax_colsum(dt, BUFP(op->a), (float*)BUFP(op->c), op->m, op->n, st);
        }
        case ENG_RMSNORM_BWD_ACC: {
            // a=x b=w d=g c=dx; tb=residual (<=0 none); sa=dw fp32 (<=0 none); sb=scratch; m=N n=D; alpha=eps
            // oa=j>0: deferred dw -- the partials stay in area j-1 of the scratch for a later COLSUM_BATCH
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * es); NEED(op->b, op->n * es); NEED(op->d, el * es); NEED(op->c, el * es);
            const void* res = nullptr; float* dw = nullptr; float* scr = nullptr;
            if (op->tb > 0) { NEED(op->tb, el * es); res = BUFP(op->tb); }
            const int defer = op->oa > 0;
            if (op->sa > 0) {
                const long long area = ax_rmsnorm_bwd_acc_scratch(op->n);
                NEED(op->sa, (long long)op->n * 4); dw = (float*)BUFP(op->sa);
                NEED(op->sb, area * (defer ? op->oa : 1)); scr = (float*)((char*)BUFP(op->sb) + (defer ? area * (op->oa - 1) : 0));
            }
            G.launches += (dw && !defer) ? 2 : 1;
            return ax_rmsnorm_bwd_acc(dt, BUFP(op->a), BUFP(op->b), BUFP(op->d), res, BUFP(op->c), dw, scr, op->m, op->n, op->alpha, st,
                                      dw ? defer : 0);
        }
        case ENG_COLSUM_BATCH: {
            // a=scratch areas, b=int32 table of destination offsets (in units of k elements), c=fp32 arena;
            // m=count, n=D, oa=first area, k=unit
            if (op->m <= 0 || op->n <= 0 || op->oa < 0 || op->k <= 0) { set_err("colsum_batch: bad shape"); return 112; }
            NEED(op->a, ax_rmsnorm_bwd_acc_scratch(op->n) * (op->oa + op->m)); NEED(op->b, (long long)(op->oa + op->m) * 4);
            NEED(op->c, 4);
            G.launches++;
            return ax_colsum_batch((const float*)BUFP(op->a), (float*)BUFP(op->c), (const int*)BUFP(op->b), op->oa, op->m, op->n, op->k,
                                   (long long)(G.bufs[op->c].bytes / 4), G.d_status, st);
        }
        case ENG_SILU_BWD: {
            const long long n = op->n;
            NEED(op->a, n * es); NEED(op->b, n * es); NEED(op->d, n * es); NEED(op->c, n * es); NEED(op->tb, n * es);
            G.launches++;
            return ax_silu_bwd(dt, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), BUFP(op->tb), n, st);
        }
        case ENG_EMBED: case ENG_EMBED_I32: {
            const long long el = (long long)op->m * op->n;
            NEED(op->b, (long long)op->m * 4); NEED(op->c, el * es); NEED(op->a, (long long)op->n * es);
            G.launches++;
            return ax_embed(dt, BUFP(op->a), BUFP(op->b), op->kind == ENG_EMBED_I32, BUFP(op->c), op->m, op->n,
                            table_rows(op->a, op->n, es), G.d_status, st);
        }
        case ENG_EMBED_BWD: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * (dt >= 1 ? 2 : 4)); NEED(op->b, (long long)op->m * 4); NEED(op->c, (long long)op->n * 4);
            G.launches++;
            return ax_embed_bwd_atomic(dt >= 1, BUFP(op->a), (const float*)BUFP(op->b), (float*)BUFP(op->c), op->m, op->n,
                                       table_rows(op->c, op->n, 4), G.d_status, st);
        }
        case ENG_EMBED_BWD_DET: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * (dt >= 1 ? 2 : 4)); NEED(op->b, (long long)op->m * 4); NEED(op->c, (long long)op->n * 4);
            G.launches++;
            return ax_embed_bwd_det(dt, BUFP(op->a), (const int*)BUFP(op->b), (float*)BUFP(op->c), op->m, op->n,
                                    table_rows(op->c, op->n, 4), G.d_status, st);
        }
        case ENG_COUNTVALID:
            NEED(op->a, (long long)op->m * 4); NEED(op->c, 4);
            G.launches++;
            return ax_countvalid((const float*)BUFP(op->a), (float*)BUFP(op->c), op->m, st);
        case ENG_CE: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * es); NEED(op->b, (long long)op->m * 4); NEED(op->c, el * es); NEED(op->d, 4);
            const float* den = nullptr;
            if (op->sa > 0) { NEED(op->sa, 4); den = (const float*)BUFP(op->sa); }
            G.launches++;
            return ax_ce(dt, BUFP(op->a), (const float*)BUFP(op->b), BUFP(op->c), (float*)BUFP(op->d), den, op->m, op->n, G.d_status, st);
        }
        case ENG_CE_FUSED: {
            // a=logits b=targets(int32) c=dlogits d=loss; sa=denom; sb=scratch (N+8 floats); m=N n=V
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * es); NEED(op->b, (long long)op->m * 4); NEED(op->c, el * es); NEED(op->d, 4);
            NEED(op->sa, 4); NEED(op->sb, ((long long)op->m + 8) * 4);
            G.launches += 2;
            return ax_ce_fused(dt, BUFP(op->a), (const int*)BUFP(op->b), BUFP(op->c), (float*)BUFP(op->d),
                               (float*)BUFP(op->sa), (float*)BUFP(op->sb), op->m, op->n, G.d_status, st);
        }
        case ENG_TICK:
            NEED(op->a, 4);
            G.launches++;
            return ax_tick((float*)BUFP(op->a), st);
        case ENG_CAST: {
            const long long n = (long long)op->m * (op->n > 0 ? op->n : 1);
            NEED(op->a, n * (op->tb == 0 ? 4 : 2)); NEED(op->c, n * (op->tb == 0 ? 2 : 4));
            G.launches++;
            return ax_cast(op->tb != 0, BUFP(op->a), BUFP(op->c), n, st);
        }
        case ENG_TRANSPOSE_BF16: {
            // a = bf16 [m,n]; c = [n,m] bf16 (dt=1) or fp32 (dt=0)
            const long long el = (long long)op->m * op->n;
            if (op->a == op->c) { set_err("transpose: in place is not supported"); return 112; }
            NEED(op->a, el * 2); NEED(op->c, el * (dt == 1 ? 2 : 4));
            G.launches++;
            return ax_transpose_bf16(dt != 1, BUFP(op->a), BUFP(op->c), op->m, op->n, st);
        }
        case ENG_ROWDOT: {
            const long long el = (long long)op->m * op->n;
            NEED(op->a, el * (dt >= 1 ? 2 : 4)); NEED(op->b, el * (dt >= 1 ? 2 : 4)); NEED(op->c, (long long)op->m * 4);
            G.launches++;
            return ax_rowdot(dt, BUFP(op->a), BUFP(op->b), (float*)BUFP(op->c), op->m, op->n, st);
        }
        case ENG_FLASH: {
            // a=q b=k d=v c=o [B,H|KV,T,DH]; m=T n=DH k=KV batch=B tb=H; sa=lse (0 none); alpha=scale
            if (dt != 1 || op->n % 16 || op->n > 128) { set_err("flash: needs bf16, head_dim %% 16 == 0, <= 128"); return 101; }
            const int T = op->m, DH = op->n, KV = op->k, B = op->batch, H = op->tb;
            if (KV <= 0 || H % KV) { set_err("flash: H %% KV != 0"); return 101; }
            NEED(op->a, (long long)B * H * T * DH * 2); NEED(op->c, (long long)B * H * T * DH * 2);
            NEED(op->b, (long long)B * KV * T * DH * 2); NEED(op->d, (long long)B * KV * T * DH * 2);
            float* lse = nullptr;
            if (op->sa > 0) { NEED(op->sa, (long long)B * H * T * 4); lse = (float*)BUFP(op->sa); }
            AttnShape s = shape_bhtd(B, H, KV, T, DH, op->alpha);
            G.launches++;
            if (!(G.fallback & 2)) {
                const int rc = ax_attn_fwd_tc(BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), lse, s, G.d_status, st);
                if (rc == 0) return 0;
                if (rc > 0) return rc;
            }
            return ax_attn_fwd_simt(1, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), lse, s, st);
        }
        case ENG_FLASH_BWD: {
            // a=q b=k d=v c=dO; sa=lse sb=D[B,T,H] tb=dq sc=dk oa=dv (fp32) ob=H; m=T n=DH k=KV batch=B
            if (dt != 1 || op->n % 16 || op->n > 128) { set_err("flash_bwd: needs bf16, head_dim %% 16 == 0, <= 128"); return 102; }
            const int T = op->m, DH = op->n, KV = op->k, B = op->batch, H = op->ob;
            if (KV <= 0 || H <= 0 || H % KV) { set_err("flash_bwd: H %% KV != 0"); return 102; }
            const long long qe = (long long)B * H * T * DH, ke = (long long)B * KV * T * DH;
            NEED(op->a, qe * 2); NEED(op->c, qe * 2); NEED(op->b, ke * 2); NEED(op->d, ke * 2);
            NEED(op->sa, (long long)B * H * T * 4); NEED(op->sb, (long long)B * H * T * 4);
            NEED(op->tb, qe * 4); NEED(op->sc, ke * 4); NEED(op->oa, ke * 4);
            AttnShape s = shape_bhtd(B, H, KV, T, DH, op->alpha);
            G.launches += 2;
            // the reference accumulates into pre-zeroed fp32 buffers; writing the full
            // sums gives the same result without atomics
            return ax_attn_bwd_simt(1, 0, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), (const float*)BUFP(op->sa),
                                    (const float*)BUFP(op->sb), BUFP(op->tb), BUFP(op->sc), BUFP(op->oa), s, st);
        }
        case ENG_ATTN_FWD: {
            // a=q [B,T,H,DH] b=k d=v [B,T,KV,DH] c=o; sa=lse [B,H,T]; m=T n=DH k=KV batch=B tb=H; alpha=scale
            const int T = op->m, DH = op->n, KV = op->k, B = op->batch, H = op->tb;
            if (KV <= 0 || H <= 0 || H % KV) { set_err("attn: H %% KV != 0"); return 101; }
            NEED(op->a, (long long)B * H * T * DH * es); NEED(op->c, (long long)B * H * T * DH * es);
            NEED(op->b, (long long)B * KV * T * DH * es); NEED(op->d, (long long)B * KV * T * DH * es);
            NEED(op->sa, (long long)B * H * T * 4);
            AttnShape s = shape_bthd(B, H, KV, T, DH, op->alpha);
            G.launches++;
            if (dt == 1 && !(G.fallback & 2)) {
                const int rc = ax_attn_fwd_tc(BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), (float*)BUFP(op->sa), s, G.d_status, st);
                if (rc == 0) return 0;
                if (rc > 0) return rc;
            }
            return ax_attn_fwd_simt(dt, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), (float*)BUFP(op->sa), s, st);
        }
        case ENG_ATTN_BWD: {
            // a=q b=k d=v c=dO; sa=lse sb=o tb=dq sc=dk oa=dv ob=H oc=D scratch [B,T,H] fp32.
            // gamma > 0: the inverse rotary of dq and dk is part of the op; beta / gamma hold the buffer
            // indices of the cos / sin tables (float-encoded like the reference's ids; sin is never slot 0)
            const int T = op->m, DH = op->n, KV = op->k, B = op->batch, H = op->ob;
            if (KV <= 0 || H <= 0 || H % KV) { set_err("attn_bwd: H %% KV != 0"); return 102; }
            const long long qe = (long long)B * H * T * DH, ke = (long long)B * KV * T * DH;
            NEED(op->a, qe * es); NEED(op->c, qe * es); NEED(op->sb, qe * es); NEED(op->b, ke * es); NEED(op->d, ke * es);
            NEED(op->sa, (long long)B * H * T * 4); NEED(op->oc, (long long)B * H * T * 4);
            NEED(op->tb, qe * es); NEED(op->sc, ke * es); NEED(op->oa, ke * es);
            const float* rc_ = nullptr; const float* rs_ = nullptr;
            if (op->gamma > 0.f) {
                const int ic = (int)op->beta, is = (int)op->gamma;
                NEED(ic, (long long)T * (DH / 2) * 4); NEED(is, (long long)T * (DH / 2) * 4);
                rc_ = (const float*)BUFP(ic); rs_ = (const float*)BUFP(is);
            }
            AttnShape s = shape_bthd(B, H, KV, T, DH, op->alpha);
            bool rotated = false;
            int done = 0;
            if (dt == 1 && !(G.fallback & 2)) {
                // the tensor-core path needs an fp32 dQ accumulator behind the D scratch in the same buffer
                const long long dwords = (long long)B * H * T;
                float* dq_acc = have(op->oc, (dwords + qe) * 4) ? (float*)BUFP(op->oc) + dwords : nullptr;
                int rc = ax_attn_bwd_tc(BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->sb), BUFP(op->c), (const float*)BUFP(op->sa),
                                        (float*)BUFP(op->oc), dq_acc, BUFP(op->tb), BUFP(op->sc), BUFP(op->oa), s, rc_, rs_, G.d_status, st);
                if (rc == 0) { rotated = rc_ != nullptr; done = 1; }
                else if (rc < 0 && rc_) {        // served without the fused rotary (head_dim 128)?
                    rc = ax_attn_bwd_tc(BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->sb), BUFP(op->c), (const float*)BUFP(op->sa),
                                        (float*)BUFP(op->oc), dq_acc, BUFP(op->tb), BUFP(op->sc), BUFP(op->oa), s, nullptr, nullptr, G.d_status, st);
                    if (rc == 0) done = 1;
                }
                if (rc > 0) return rc;
                if (done) G.launches += 4;
            }
            if (!done) {
                G.launches += 3;
                int rc = ax_rowdot(dt, BUFP(op->c), BUFP(op->sb), (float*)BUFP(op->oc), (long long)B * T * H, DH, st);
                if (rc) return rc;
                rc = ax_attn_bwd_simt(dt, dt == 1 ? 1 : 0, BUFP(op->a), BUFP(op->b), BUFP(op->d), BUFP(op->c), (const float*)BUFP(op->sa),
                                      (const float*)BUFP(op->oc), BUFP(op->tb), BUFP(op->sc), BUFP(op->oa), s, st);
                if (rc) return rc;
            }
            if (rc_ && !rotated) {
                G.launches++;
                return ax_rope2(dt, BUFP(op->tb), rc_, rs_, BUFP(op->tb), T, DH, (long long)B * T * H, H, 1,
                                BUFP(op->sc), BUFP(op->sc), (long long)B * T * KV, KV, st);
            }
            return 0;
        }
        case ENG_L2ACC:
            NEED(op->a, (long long)op->n * 4); NEED(op->c, 4);
            G.launches++;
            return ax_l2acc((const float*)BUFP(op->a), (float*)BUFP(op->c), op->n, st);
        case ENG_CLIPSCALE:
            NEED(op->a, 4); NEED(op->c, 4);
            G.launches++;
            return ax_clipscale((const float*)BUFP(op->a), (float*)BUFP(op->c), op->alpha, st);
        case ENG_GNORM_FLAT: {
            // a=grad arena, c=partials scratch, m=chunks (AX_ADAMW_CHUNK elements each), oa=chunk offset in a,
            // d=scalar out buffer with index ob, tb=step counter to tick (<=0 none)
            const long long n = (long long)op->m * AX_ADAMW_CHUNK, off = (long long)op->oa * AX_ADAMW_CHUNK;
            const long long np = (n + AX_GNORM_CHUNK - 1) / AX_GNORM_CHUNK;
            NEED(op->a, (off + n) * 4); NEED(op->c, (np > 0 ? np : 1) * 4); NEED(op->d, ((long long)op->ob + 1) * 4);
            float* tick = nullptr;
            if (op->tb > 0) { NEED(op->tb, 4); tick = (float*)BUFP(op->tb); }
            G.launches += 2;
            return ax_gnorm_flat((const float*)BUFP(op->a) + off, (float*)BUFP(op->c), n, tick, (float*)BUFP(op->d) + op->ob, st);
        }
        case ENG_ADAMW_FLAT: {
            // a=master b=grad c=m d=v (a,c,d segment-local; b, mirror and flags offset by k chunks);
            // sa=bf16 mirror (<=0 none) sb=lr tb=t sc=decay flags oa=partials ob=#partials oc=norm out (<=0 none)
            const long long n = (long long)op->m * AX_ADAMW_CHUNK, off = (long long)op->k * AX_ADAMW_CHUNK;
            NEED(op->a, n * 4); NEED(op->c, n * 4); NEED(op->d, n * 4); NEED(op->b, (off + n) * 4);
            NEED(op->sb, 4); NEED(op->tb, 4); NEED(op->sc, (long long)op->k + op->m);
            void* pbf = nullptr; float* gout = nullptr; const float* parts = nullptr;
            if (op->sa > 0) { NEED(op->sa, (off + n) * 2); pbf = (char*)BUFP(op->sa) + off * 2; }
            if (op->ob > 0) { NEED(op->oa, (long long)op->ob * 4); parts = (const float*)BUFP(op->oa); }
            if (op->oc > 0) { NEED(op->oc, 4); gout = (float*)BUFP(op->oc); }
            G.launches++;
            return ax_adamw_flat((float*)BUFP(op->a), (const float*)BUFP(op->b) + off, (float*)BUFP(op->c), (float*)BUFP(op->d),
                                 pbf, (const unsigned char*)BUFP(op->sc) + op->k, (const float*)BUFP(op->tb), (const float*)BUFP(op->sb),
                                 parts, op->ob > 0 ? op->ob : 0, gout, op->alpha, op->beta, op->gamma, n, st);
        }
        // ── collectives ──
        case ENG_ALLREDUCE: case ENG_REDUCE: case ENG_BROADCAST: {
            // n = element count, or (m chunks of AX_ADAMW_CHUNK elements at chunk offset oa) when m > 0
            if (!G.comm) { set_err("collective before nccl_init"); return 104; }
            const bool half = op->kind == ENG_BROADCAST && dt == 1;
            const long long e = half ? 2 : 4;
            const long long cnt = op->m > 0 ? (long long)op->m * AX_ADAMW_CHUNK : op->n;
            const long long off = op->m > 0 ? (long long)op->oa * AX_ADAMW_CHUNK : 0;
            NEED(op->a, (off + cnt) * e);
            char* p = (char*)BUFP(op->a) + off * e;
            G.launches++;
            if (op->kind == ENG_ALLREDUCE) return nccl_wait(ncclAllReduce(p, p, cnt, ncclFloat, ncclAvg, G.comm, st));
            if (op->tb < 0 || op->tb >= G.world) { set_err("collective root %d outside world %d", op->tb, G.world); return 112; }
            if (op->kind == ENG_REDUCE) return nccl_wait(ncclReduce(p, p, cnt, ncclFloat, ncclAvg, op->tb, G.comm, st));
            return nccl_wait(ncclBroadcast(p, p, cnt, half ? ncclBfloat16 : ncclFloat, op->tb, G.comm, st));
        }
        case ENG_ALLGATHER_F32: {
            if (!G.comm) { set_err("collective before nccl_init"); return 104; }
            NEED(op->a, (long long)(op->oa + op->n) * 4); NEED(op->c, (long long)op->n * G.world * 4);
            G.launches++;
            return nccl_wait(ncclAllGather((const float*)BUFP(op->a) + op->oa, BUFP(op->c), op->n, ncclFloat, G.comm, st));
        }
        case ENG_GROUP:
            if (!G.comm) { set_err("group before nccl_init"); return 104; }
            return op->tb ? nccl_wait(ncclGroupEnd()) : nccl_wait(ncclGroupStart());
        case ENG_FORK: case ENG_JOIN: {
            // FORK: the comm stream waits for everything queued on the main stream so far.
            // JOIN: the main stream waits for everything queued on the comm stream so far.
            if (G.fork_used >= G.fork_events.size()) {
                cudaEvent_t e;
                if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming)) return 113;
                G.fork_events.push_back(e);
            }
            cudaEvent_t e = G.fork_events[G.fork_used++];
            cudaStream_t from = op->kind == ENG_FORK ? G.stream : G.comm_stream;
            cudaStream_t to = op->kind == ENG_FORK ? G.comm_stream : G.stream;
            if (cudaEventRecord(e, from)) return 113;
            if (cudaStreamWaitEvent(to, e, 0)) return 113;
            return 0;
        }
        case ENG_STREAM:
            G.cur = op->tb == 2 ? G.side_stream : (op->tb ? G.comm_stream : G.stream);
            ax_gemm_side(G.cur != G.stream);
            return 0;
        case ENG_EVENT: {
            // tb=1: record event oa on stream sa; tb=2: stream sa waits for event oa (sa: 0 main, 1 collectives, 2 side)
            if (op->oa < 0 || op->oa >= 65536 || op->sa < 0 || op->sa > 2 || (op->tb != 1 && op->tb != 2)) { set_err("event: bad arguments"); return 112; }
            if ((size_t)op->oa >= G.named_events.size()) G.named_events.resize(op->oa + 1, nullptr);
            cudaEvent_t& e = G.named_events[op->oa];
            if (!e && cudaEventCreateWithFlags(&e, cudaEventDisableTiming)) { e = nullptr; return 113; }
            cudaStream_t s = op->sa == 2 ? G.side_stream : (op->sa ? G.comm_stream : G.stream);
            if (op->tb == 1) return cudaEventRecord(e, s) ? 113 : 0;
            return cudaStreamWaitEvent(s, e, 0) ? 113 : 0;
        }
        default:
            set_err("unknown op kind %d", op->kind);
            return 100;
    }
}

static int run_ops(const EngOp* ops, int n_ops) {
    G.fork_used = 0;
    G.cur = G.stream;
    ax_gemm_side(0);
    for (int i = 0; i < n_ops; i++) {
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        const bool prof = G.profile && ops[i].kind >= 0 && ops[i].kind < ENG_KIND_COUNT &&
                          ops[i].kind != ENG_GROUP && ops[i].kind != ENG_STREAM && ops[i].kind != ENG_FORK && ops[i].kind != ENG_JOIN &&
                          ops[i].kind != ENG_EVENT;
        if (prof) { cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventRecord(e0, G.cur); }
        int rc = exec_op(&ops[i]);
        if (!rc) {
            cudaError_t ce = cudaPeekAtLastError();
            if (ce != cudaSuccess) { set_err("op %d (kind %d): %s", i, ops[i].kind, cudaGetErrorString(ce)); cudaGetLastError(); rc = 130; }
        }
        if (prof) {
            cudaEventRecord(e1, G.cur); cudaEventSynchronize(e1);
            float ms = 0.f; cudaEventElapsedTime(&ms, e0, e1);
            G.prof_ms[ops[i].kind] += ms; G.prof_calls[ops[i].kind]++;
            cudaEventDestroy(e0); cudaEventDestroy(e1);
        }
        if (rc) {                      // a failed plan leaves nothing noted for a later one
            g_xseg = {}; g_lgrad.n = 0;
            G.last_op_rc = rc; G.cur = G.stream; return 1000 + i;
        }
    }
    G.cur = G.stream;
    return 0;
}

API int eng_run_plan(const EngOp* ops, int n_ops, int sync) {
    if (!G.inited) { set_err("engine not initialised"); return 1; }
    int rc = run_ops(ops, n_ops);
    if (rc) return rc;
    return sync ? eng_sync() : 0;
}

API int eng_capture_plan(const EngOp* ops, int n_ops) {
    if (!G.inited) { set_err("engine not initialised"); return 1; }
    if (G.graph) { cudaGraphExecDestroy(G.graph); G.graph = nullptr; }
    eng_sync();
    const int prof = G.profile; G.profile = 0;
    if (cudaStreamBeginCapture(G.stream, cudaStreamCaptureModeThreadLocal)) { G.profile = prof; set_err("begin capture failed"); return 1; }
    const long long before = G.launches;
    int rc = run_ops(ops, n_ops);
    G.profile = prof;
    cudaGraph_t graph = nullptr;
    cudaError_t ce = cudaStreamEndCapture(G.stream, &graph);
    G.graph_launches = G.launches - before;
    G.launches = before;
    if (rc) { if (graph) cudaGraphDestroy(graph); cudaGetLastError(); return rc; }
    if (ce != cudaSuccess) { set_err("end capture: %s", cudaGetErrorString(ce)); cudaGetLastError(); return 2; }
    ce = cudaGraphInstantiate(&G.graph, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) { set_err("instantiate: %s", cudaGetErrorString(ce)); cudaGetLastError(); G.graph = nullptr; return 3; }
    return 0;
}

API int eng_replay(int times, int sync) {
    if (!G.graph) { set_err("no captured plan"); return 1; }
    for (int i = 0; i < times; i++) {
        if (cudaGraphLaunch(G.graph, G.stream)) { set_err("graph launch failed: %s", cudaGetErrorString(cudaGetLastError())); return 2; }
        G.launches += G.graph_launches;
    }
    return sync ? eng_sync() : 0;
}

API int eng_time_replay(int times, float* ms_out) {
    if (!G.graph) { set_err("no captured plan"); return 1; }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, G.stream);
    int rc = 0;
    for (int i = 0; i < times && !rc; i++) {
        if (cudaGraphLaunch(G.graph, G.stream)) { set_err("graph launch failed: %s", cudaGetErrorString(cudaGetLastError())); rc = 2; }
        G.launches += G.graph_launches;
    }
    cudaEventRecord(e1, G.stream);
    if (cudaEventSynchronize(e1) && !rc) { set_err("replay failed: %s", cudaGetErrorString(cudaGetLastError())); rc = 130; }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (ms_out) *ms_out = ms;
    return rc;
}

API int eng_time_plan(const EngOp* ops, int n_ops, int reps, int flush_l2, float* ms_out) {
    if (!G.inited) return 1;
    if (reps < 1) reps = 1;
    const size_t FL = 256u << 20;
    if (flush_l2 && !G.l2_flush && cudaMalloc(&G.l2_flush, FL)) { G.l2_flush = nullptr; cudaGetLastError(); set_err("flush buffer alloc failed"); return 2; }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    double total = 0.0;
    int rc = 0;
    for (int r = 0; r < reps && !rc; r++) {
        if (flush_l2) cudaMemsetAsync(G.l2_flush, r & 0xff, FL, G.stream);
        cudaEventRecord(e0, G.stream);
        rc = run_ops(ops, n_ops);
        cudaEventRecord(e1, G.stream);
        if (cudaEventSynchronize(e1)) rc = rc ? rc : 130;
        float ms = 0.f; cudaEventElapsedTime(&ms, e0, e1);
        total += ms;
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (ms_out) *ms_out = (float)(total / reps);
    return rc;
}

API int eng_profile(int on) {
    G.profile = on;
    if (on) { memset(G.prof_ms, 0, sizeof(G.prof_ms)); memset(G.prof_calls, 0, sizeof(G.prof_calls)); }
    return 0;
}
API int eng_profile_read(float* ms, int* calls, int n) {
    for (int i = 0; i < n && i < ENG_KIND_COUNT; i++) { ms[i] = G.prof_ms[i]; calls[i] = G.prof_calls[i]; }
    return 0;
}
