/* C ABI of the B200 2-simplicial attention library (libsimplicial_attn_b200.so).
 *
 * The operator:  logits_ijk = scale * sum_d Q_id * K1_jd * (K2_kd + k2_bias)
 *                over the causal windows  j in (i-w1, i],  k in (i-w2, i];
 *                P = softmax over each query's (j,k) pairs;
 *                O_i = sum_jk P_ijk * V1_j * (V2_k + v2_bias);   LSE_i = log sum_jk exp(logits_ijk).
 *
 * Every entry point takes plain pointers and sizes, allocates nothing, launches on the caller's
 * stream, never synchronises the host (except sa_read_status) and returns an sa_status.
 * All buffers -- inputs, outputs, LSE and workspace -- are owned by the caller and live in device
 * memory of the current CUDA device.
 *
 * Logical tensor shapes (the reference's, simplicial/reference.py:16-18): Q, O, dO, dQ are
 * [B, N, H, D]; K1, V1, dK1, dV1 are [B, N + halo1, Hkv, D]; K2, V2, dK2, dV2 are
 * [B, N + halo2, Hkv, D]; LSE is [B, H, N] fp32 contiguous.  Any (b, n, h) element strides are
 * accepted, the d stride is 1.  H % Hkv == 0 and query head h reads KV head h / (H / Hkv).
 * halo1/halo2 count extra leading K/V rows that precede query row 0 (a sequence shard's halo);
 * query row n pairs with K1 row n + halo1 and K2 row n + halo2; windows are clipped at row 0.
 */
#ifndef SIMPLICIAL_ATTN_B200_H
#define SIMPLICIAL_ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    SA_OK = 0,
    SA_ERR_NULL_POINTER = 1,     /* a required pointer is NULL */
    SA_ERR_BAD_SHAPE = 2,        /* non-positive extent, H % Hkv != 0, negative halo, window < 1 */
    SA_ERR_BAD_STRIDE = 3,       /* a stride breaks the 16-byte alignment the kernels need */
    SA_ERR_UNSUPPORTED = 4,      /* dtype / head dim / window outside what the chosen kernel handles */
    SA_ERR_WORKSPACE = 5,        /* workspace too small or misaligned (256 bytes) */
    SA_ERR_LAUNCH = 6,           /* CUDA reported an error at launch */
    SA_ERR_DEVICE_TIMEOUT = 7,   /* a bounded device-side wait gave up (seen through sa_read_status) */
    SA_ERR_NOT_SM100 = 8         /* the current device is not compute capability 10.x */
} sa_status;

typedef enum { SA_BF16 = 0, SA_F16 = 1, SA_F32 = 2 } sa_dtype;

/* Kernel family.  AUTO picks the tcgen05 kernels whenever they cover the problem (bf16 or fp16, D in
 * {64,128}, effective w2 <= 1024; a K2 window wider than 128 positions is processed in passes over
 * 128-position chunks whose results are merged, with temporaries in the workspace) and the general
 * kernels otherwise.  The general kernels are plain
 * CUDA-core fp32 code for every dtype, head dim and window; they also serve as the on-device
 * cross-check of the tensor-core kernels. */
typedef enum { SA_ALGO_AUTO = 0, SA_ALGO_GENERAL = 1, SA_ALGO_TCGEN05 = 2 } sa_algo;

/* (b, n, h) element strides of one tensor; the innermost (d) stride is 1. */
typedef struct { int64_t b, n, h; } sa_strides;

typedef struct {
    int32_t B, N, H, Hkv, D;
    int32_t w1, w2;              /* window sizes, >= 1 (values above the row count are clipped) */
    int32_t halo1, halo2;        /* leading halo rows of K1/V1 and of K2/V2 */
    int32_t dtype;               /* sa_dtype of every tensor except LSE */
    int32_t algo;                /* sa_algo */
    float scale, k2_bias, v2_bias;
    sa_strides q, k1, k2, v1, v2, o;          /* forward tensors (o also describes O in backward) */
    sa_strides d_o, dq, dk1, dk2, dv1, dv2;   /* backward tensors (ignored by sa_forward) */
} sa_params;

/* Replaces the launch of two_simplicial_attn_fwd_kernel in
 * TwoSimplicialAttentionFunction.forward (simplicial/triton_impl.py:19-58; kernel
 * simplicial/kernels.py:11-171).  Writes O (dtype) and LSE (fp32, natural log; the reference's
 * `M`, simplicial/kernels.py:164-167).  `workspace` must hold sa_forward_workspace_size() bytes,
 * 256-byte aligned; its first 256 bytes hold the device status word and must be zero before the
 * first call that uses the buffer (the library never clears them except in sa_read_status). */
int sa_forward(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1,
               const void* v2, void* o, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces compute_D_kernel plus the two backward launches of
 * TwoSimplicialAttentionFunction.backward (simplicial/triton_impl.py:61-158; kernels
 * simplicial/kernels.py:175-382, :386-566, :569-571).  Any of dq, dk1, dk2, dv1, dv2 may be NULL
 * (gradient not needed, the reference's needs_input_grad gating, triton_impl.py:73-77).  Outputs
 * are overwritten, not accumulated into, and are written without atomics in a fixed order. */
int sa_backward(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1,
                const void* v2, const void* o, const float* lse, const void* d_o, void* dq, void* dk1,
                void* dk2, void* dv1, void* dv2, void* workspace, size_t workspace_bytes, void* stream);

/* The same backward for callers that have no way to obtain a device workspace at the moment they
 * need the gradients.  Typical cases: a plugin that runs inside a host framework's memory-allocator
 * callback, where calling the allocator again would re-enter it or deadlock; a worker in a process
 * whose device memory was handed out in full to a pool that somebody else owns, so that a cudaMalloc
 * fails; a real-time loop that is not allowed to take the allocation lock at all.  It has no
 * counterpart in the reference.  Instead of a caller workspace the call uses a 32 MiB scratch array
 * that is part of the library image -- every GPU that loads the library gives up that much memory
 * until the process exits -- and it calls no cudaMalloc, cudaFree or any other allocating routine.
 * Problems whose sa_backward_workspace_size() exceeds sa_backward_static_capacity() are rejected
 * with SA_ERR_WORKSPACE (at D=128, w2=32 the limit is about 30 000 query rows summed over batch and
 * heads).  The first call on each device looks up the array's device address, with that device
 * current; make that first call before any stream capture begins.  All calls on a device share the
 * one array and find in it whatever the previous call left: two calls whose kernels may overlap on
 * the GPU (different streams with no ordering between them) race on it, so keep them ordered.
 * The array's first bytes hold the device status word.  It is zero when the library is loaded and
 * the call does not clear it, so a timeout recorded by an earlier call stays visible until
 * sa_read_status_static() reports and clears it. */
int sa_backward_static(const sa_params* p, const void* q, const void* k1, const void* k2, const void* v1,
                       const void* v2, const void* o, const float* lse, const void* d_o, void* dq, void* dk1,
                       void* dk2, void* dv1, void* dv2, void* stream);
size_t sa_backward_static_capacity(void);

/* sa_read_status() for the built-in scratch array of sa_backward_static(): synchronises `stream`,
 * returns SA_OK or SA_ERR_DEVICE_TIMEOUT and clears the word.  Call it after the calls whose result
 * you are about to trust.  No counterpart in the reference. */
int sa_read_status_static(void* stream);

/* Workspace sizes in bytes for the given problem (the reference allocates its work buffers inside
 * the autograd function, triton_impl.py:23-25,73-77; here the caller does).  Never 0: the first
 * 256 bytes hold the device status word.  The sizes depend on the windows (a K2 window wider than
 * 128 positions needs room for one more O / LSE, or one more set of gradients). */
size_t sa_forward_workspace_size(const sa_params* p);
size_t sa_backward_workspace_size(const sa_params* p);

/* Synchronises `stream` and returns the status word the kernels of earlier calls left in
 * `workspace` (SA_OK or SA_ERR_DEVICE_TIMEOUT), then clears it.  The reference has no
 * counterpart: its failures surface as Triton exceptions. */
int sa_read_status(void* workspace, void* stream);

/* Reads the status word without synchronising anything: copies it (16 bytes) from `workspace` to
 * `device_slot` on `stream`, and from there to `host_slot` (pinned host memory) on `side_stream`, which
 * waits for the first copy through `ev_ready`; `ev_done` is recorded behind the second copy.  Once
 * `ev_done` has completed, `host_slot` holds {code, wait site, block, 0} as four ints.  The workspace
 * is free for reuse as soon as `stream` has passed the first copy, and `stream` never waits for the
 * transfer to the host.  Streams, events and both slots are the caller's.  No counterpart in the
 * reference. */
int sa_status_relay(const void* workspace, void* device_slot, void* host_slot, void* stream, void* side_stream,
                    void* ev_ready, void* ev_done);

/* sa_read_status(), also returning where the wait gave up: `where` receives the id of the wait site inside
 * the kernel and `block` the index of the thread block that recorded it (either may be NULL). */
int sa_read_status_ex(void* workspace, void* stream, int* where, int* block);

/* Every wait inside the kernels (on an mbarrier that another warp, the TMA unit or the tensor cores
 * complete) is bounded: when it lasts longer than the limit the block records
 * SA_ERR_DEVICE_TIMEOUT in the status word, stops waiting and returns, so the context stays usable.
 * The limit is 2 s unless changed here (0 restores the default); it applies to calls made afterwards,
 * process-wide.  No counterpart in the reference. */
void sa_set_wait_limit_ns(uint64_t limit_ns);

/* Self-test of that mechanism: launches one warp that waits, with the given limit (at most 0.1 s),
 * on a barrier nobody arrives on.  The kernel returns by itself once the limit has passed; afterwards
 * sa_read_status(workspace) reports SA_ERR_DEVICE_TIMEOUT.  `workspace` needs 256 bytes, 256-byte
 * aligned, zero status word.  Nothing faults, traps or spins without a bound. */
int sa_selftest_wait_timeout(void* workspace, uint64_t limit_ns, void* stream);

/* Which kernel family AUTO resolves to for `p` (SA_ALGO_GENERAL or SA_ALGO_TCGEN05), or a negative
 * sa_status if `p` is invalid. */
int sa_resolve_algo(const sa_params* p);

/* Strided copy between host and device (either direction, or device to device) on `stream`: `rows`
 * pieces of `row_bytes` bytes, `src_pitch` / `dst_pitch` bytes apart.  Used to move one group of
 * heads of a [B, N, H, D] tensor that lives in pinned host memory without staging it first.  Host
 * memory must be pinned for the copy to overlap with kernels.  No counterpart in the reference
 * (its tensors never leave the device). */
int sa_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                       size_t rows, void* stream);

/* Number of kernels this library has launched in this process so far (all devices, all streams).
 * No counterpart in the reference. */
uint64_t sa_kernel_launches(void);

const char* sa_strerror(int status);
int sa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SIMPLICIAL_ATTN_B200_H */
