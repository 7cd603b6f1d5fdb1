/* axeng.h — C ABI of libaxeng.so, the B200 (sm_100a) engine for the compiled
 * training step.
 *
 * The first twelve entry points are what the reference's ctypes binding loads
 * (axis/engine.py:81-100) and what its CUDA runtime exports
 * (axis/_csrc/runtime.cu:814-876, 1166-1197): same names, argument meaning and
 * integer return codes, so the reference's own Python (`axis.engine.Engine`,
 * `axis.compile.CompiledTransformer`) can load this library unchanged.  The
 * entry points after them are additions used by this repository's host code.
 *
 * Process-global, single engine per process, one GPU per process, not thread
 * safe — as in the reference (axis/_csrc/runtime.cu:57-65).  All device memory
 * is owned by the library.  Host pointers are borrowed for the duration of a
 * call only.  There is no CPU fallback: every entry point needs a CUDA device.
 */
#ifndef AXENG_H
#define AXENG_H

#ifdef __cplusplus
extern "C" {
#endif

/* Op descriptor: 17 int32 + 3 float = 80 bytes, field order fixed
 * (axis/_csrc/runtime.cu:46-55, axis/engine.py:24-35). */
typedef struct EngOp {
    int   kind;
    int   a, b, c, d;          /* buffer indices, -1 = none                   */
    int   m, n, k;
    int   batch, tb;
    int   sa, sb, sc;          /* strides, or extra buffer indices (0 = none) */
    int   dt;                  /* 0 fp32 | 1 bf16 | 2 bf16 in, fp32 out       */
    int   oa, ob, oc;          /* element offsets, or extra operands          */
    float alpha, beta, gamma;
} EngOp;

/* Op kinds 0..31 are the reference's (axis/_csrc/runtime.cu:35-44); kinds from
 * 32 up are fused ops of this engine (see axis_b200/engine.py for role maps). */
enum EngOpKind {
    ENG_GEMM = 0, ENG_ADD = 1, ENG_MUL = 2, ENG_SILU_MUL = 3, ENG_RMSNORM = 4,
    ENG_ADAMW = 5, ENG_SCALE = 6, ENG_COPY = 7, ENG_GEMM_SB = 8, ENG_PERM_0213 = 9,
    ENG_ROPE = 10, ENG_SOFTMAX_CAUSAL = 11, ENG_REPEAT_KV = 12, ENG_RMSNORM_BWD = 13,
    ENG_COLSUM = 14, ENG_REPEAT_KV_BWD = 15, ENG_SOFTMAX_BWD = 16, ENG_SILU_BWD = 17,
    ENG_EMBED = 18, ENG_EMBED_BWD = 19, ENG_CE = 20, ENG_TICK = 21, ENG_CAST = 22,
    ENG_FLASH = 23, ENG_ROWDOT = 24, ENG_FLASH_BWD = 25, ENG_ALLREDUCE = 26,
    ENG_GROUP = 27, ENG_L2ACC = 28, ENG_CLIPSCALE = 29, ENG_COUNTVALID = 30,
    ENG_BROADCAST = 31,
    /* fused kinds */
    ENG_GEMM_EX = 32,         /* GEMM with a separate addend: c = alpha*op(a)op(b) + beta*d */
    ENG_ROPE_BTHD = 33,       /* rotary on the [B,T,H,DH] layout, in place allowed          */
    ENG_ATTN_FWD = 34,        /* causal GQA attention on [B,T,H,DH], saves LSE              */
    ENG_ATTN_BWD = 35,        /* dq/dk/dv on [B,T,H,DH], group-summed, no atomics           */
    ENG_RMSNORM_BWD_ACC = 36, /* dx (+ residual) and dw in one pass                         */
    ENG_CE_FUSED = 37,        /* count + loss + dlogits (in place), deterministic           */
    ENG_EMBED_BWD_DET = 38,   /* ordered scatter-add without atomics                        */
    ENG_GNORM_FLAT = 39,      /* sum of squares of a flat grad arena (+ step tick)          */
    ENG_ADAMW_FLAT = 40,      /* clip + AdamW over a flat arena with a decay-flag table     */
    ENG_EMBED_I32 = 41,       /* embedding gather with int32 ids                            */
    ENG_REDUCE = 42,          /* NCCL reduce (average) to a root rank                       */
    ENG_ALLGATHER_F32 = 43,   /* NCCL all-gather of per-rank scalars                        */
    ENG_FORK = 44,            /* side-stream fork: comm stream waits for the main stream    */
    ENG_JOIN = 45,            /* main stream waits for the comm stream                      */
    ENG_STREAM = 46,          /* tb=1: following ops go to the comm stream, tb=0: main      */
    ENG_SILU_MUL_BWD_RC = 47, /* SwiGLU backward that also rewrites h for recompute-free dW */
    ENG_GEMM_GROUP = 48,      /* 2-3 GEMMs of a layer as one launch: shared input, or one output summed over K-segments */
    ENG_TRANSPOSE_BF16 = 49,  /* c[n,m] = a[m,n]^T, a bf16; c bf16 (dt=1) or widened to fp32 (dt=0): checkpoint weights
                                 stored [out,in] in bf16 go to the [in,out] compute / master layout on the device */
    ENG_COLSUM_BATCH = 50,    /* dw of several RMSNORM_BWD_ACC launches whose partial sums were left in scratch (oa > 0 there) */
    ENG_EVENT = 51,           /* cross-stream dependency by id: record on a stream / make a stream wait (main, collectives, side) */
    ENG_GEMM_XSEG = 52,       /* extra operands of the NEXT GEMM_GROUP (no launch): a low-rank term per output (mode 1), further
                                 K-segments and a residual addend (mode 2) */
    ENG_LORA_GRAD = 53,       /* adapter weight gradients alpha * X^T S of up to three projections: X read once, fixed summation order */
    ENG_LORA_PROJ = 54,       /* the skinny products of adapters, x A (forward) or g B^T (backward), of up to three projections */
    ENG_KIND_COUNT
};

/* ── the reference's entry points ─────────────────────────────────────────── */

/* Create stream and handles, opt in to large shared memory, clear the buffer
 * table.  Re-entrant: a second call releases everything the first one made.
 * 0 = ok, 1..6 = failing stage.            (axis/_csrc/runtime.cu:814-834) */
int eng_init(void);

/* cudaMalloc(nelems*elsize) into slot idx; contents undefined.
 * 1 = bad index, 2 = out of memory.        (axis/_csrc/runtime.cu:836-840) */
int eng_alloc(int idx, long long nelems, int elsize);

/* 1 when fused flash attention is available (always, here).  (:842-848) */
int eng_has_flash(void);

/* NCCL bootstrap: 128-byte unique id; moving it between ranks is the
 * caller's job.                            (axis/_csrc/runtime.cu:851-865) */
int eng_nccl_id(void* out128);
int eng_nccl_init(int rank, int world, const void* id128);

/* Copies in 4-byte units on the engine stream.  Upload stages the host data
 * before returning, so the caller may free it at once; download synchronises.
 *                                          (axis/_csrc/runtime.cu:867-876) */
int eng_upload(int idx, const float* host, long long nfloats);
int eng_download(int idx, float* host, long long nfloats);

/* Execute ops in order.  First failing op i -> 1000+i (the per-op code is
 * kept for eng_last_error).  Per-op codes: 100 unknown kind, 101/102 flash
 * constraints, 104 communicator not initialised, 110 bad buffer reference,
 * 111 operand exceeds its buffer.          (axis/_csrc/runtime.cu:1166-1172) */
int eng_run_plan(const EngOp* ops, int n_ops, int sync);

/* Capture the plan into one CUDA graph (replaces an earlier one) / launch it.
 * capture: 1 begin failed, 2 end failed, 3 instantiate failed, 1000+i op i.
 * replay: 1 nothing captured, 2 launch failed.  (:1174-1191) */
int eng_capture_plan(const EngOp* ops, int n_ops);
int eng_replay(int times, int sync);

int eng_sync(void);
/* TF32 switch of the reference's cuBLAS handle.  fp32 GEMMs here always use
 * true fp32 FMA accumulation; the call is accepted and recorded.  (:1195) */
int eng_set_tf32(int on);

/* ── additions (no counterpart in the reference) ──────────────────────────── */

/* Slot idx becomes a window of `parent` starting at byte_offset (not owned). */
int eng_alloc_view(int idx, int parent, long long byte_offset, long long nbytes);
/* Zero-filled allocation. */
int eng_alloc_zero(int idx, long long nbytes);
/* Byte-granular copies with a destination/source byte offset. */
int eng_upload_raw(int idx, long long byte_offset, const void* host, long long nbytes);
int eng_download_raw(int idx, long long byte_offset, void* host, long long nbytes);
/* int64 tokens -> device int32 (values are range-checked against `limit`:
 * a token >= limit or < -1 returns 3).  */
int eng_upload_tokens(int idx, const long long* host, long long n, long long limit);
/* Read-back that does not stall the host: eng_download_async queues a copy of nfloats (<= 64) floats of buffer
 * idx into a pinned slot behind the work queued so far and returns a ticket (>= 0; negative = failure);
 * eng_download_wait blocks until that copy has landed and hands it out (4 = the ticket is unknown or older
 * than the 8 slots of the ring).  A host loop that reads step i's loss after launching step i+1 keeps the GPU
 * queue non-empty while it prepares the next batch. */
int eng_download_async(int idx, long long nfloats);
int eng_download_wait(int ticket, float* host, long long nfloats);
/* Release every buffer, graph, communicator and stream. */
int eng_shutdown(void);
/* Text of the last failure (static storage). */
const char* eng_last_error(void);
/* Device status word: 0 = clean; non-zero = a bounded device-side wait gave
 * up (code identifies the kernel).  Reading clears it when clear != 0. */
int eng_device_status(int clear);
/* Time `reps` executions of a plan with CUDA events on the engine stream,
 * flushing L2 between repetitions when flush_l2 != 0; ms_out = mean ms. */
int eng_time_plan(const EngOp* ops, int n_ops, int reps, int flush_l2, float* ms_out);
/* `times` launches of the captured graph between two CUDA events on the engine
 * stream; ms_out = total milliseconds. */
int eng_time_replay(int times, float* ms_out);
/* Per-kind accounting: when on, every op in run_plan is bracketed by events.
 * eng_profile_read fills ms[ENG_KIND_COUNT] and calls[ENG_KIND_COUNT]. */
int eng_profile(int on);
int eng_profile_read(float* ms, int* calls, int n);
/* Number of kernels / library calls launched since the last reset. */
long long eng_launch_count(int reset);
/* NCCL bootstrap with a deadline in ms (non-blocking init, polled). 0 = ok,
 * 7 = timed out, other = NCCL error. */
int eng_nccl_init_timeout(int rank, int world, const void* id128, int timeout_ms);
/* Kernel selection overrides (bit mask): 1 = general GEMM instead of tensor-core GEMM,
 * 2 = general attention, 4 = single-CTA tensor-core GEMM only, 8 = paired-CTA GEMM
 * whenever the shape allows. */
int eng_set_fallback(int mask);
/* Bytes currently allocated through eng_alloc*. */
long long eng_bytes_allocated(void);
/* Code of the kernel variant the last GEMM / cross-entropy op ran on (no counterpart in the reference; lets a
 * test assert that a shape was served by the kernel it means to check): 0x10 cross-entropy streaming rows,
 * 0x11 register-resident rows; 0x20 general GEMM, 0x21 single-CTA tcgen05 GEMM, 0x22 paired-CTA tcgen05 GEMM,
 * the GEMM codes plus 0x100 times the split-K factor. */
int eng_last_variant(void);

/* Fused RMSNorm backward that allocates nothing (no counterpart in the
 * reference).  dx = (res ? res : 0) + d(rmsnorm)/dx, dw = sum over rows of
 * g * x * inv_rms, on caller-owned DEVICE pointers, enqueued on `stream`
 * (a cudaStream_t; NULL = default stream).  x, g, res, dx: [rows, dim] in the
 * storage type dt (0 = fp32, 1 = bf16); w: [dim] in dt; dw: [dim] fp32 or NULL;
 * res may be NULL.  It needs no eng_init and no engine buffer.
 *
 * Who needs it: callers that must not allocate on the device — code running
 * while a stream is being captured into a CUDA graph, hosts that give the
 * library a fixed memory budget, and loops that cannot afford an allocator call
 * and the synchronisation it implies.  The scratch that the reduction of dw
 * needs (per-block column partials) lives in a static device array inside the
 * library instead of a caller-provided buffer: 296 x 8192 floats, about 9.7 MB,
 * resident on every GPU that loads the library until the process exits.
 *
 * Limits and rules: dim <= 8192 (larger: returns 201 and prints a message to
 * stderr).  The first call on a device looks up the array's address once
 * (with that device current); make that first call before starting any stream
 * capture.  Every call uses the same array and leaves its partials there;
 * nothing in it has to be cleared between calls, but two calls that overlap on
 * the GPU (different streams, no ordering) race on it — serialise them.
 * rows == 0 is served: dw (if given) is set to zero, dx is not touched.  The
 * call clears this thread's pending CUDA error before it launches, so 204
 * reports only its own launch.
 * Returns 0, or 201 dim too large, 202 bad argument, 203 device/symbol lookup
 * failed, 204 launch failed. */
int eng_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* g, const void* res, void* dx, float* dw,
                            int rows, int dim, int dt, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AXENG_H */
