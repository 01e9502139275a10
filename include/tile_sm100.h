/* tile_sm100.h — C ABI of libtile_sm100, the sm_100a (B200) implementation of
 * tile-rs's matmul / row-softmax / fused-attention hot path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int32 status (TSM100_OK == 0) and never throws or aborts.  On failure a
 * human-readable message is kept per thread and read with tsm100_last_error().
 * There is no CPU fallback: without a CUDA device every compute and runtime
 * entry point returns TSM100_ERR_NO_DEVICE.
 *
 * The comment on each declaration names the reference interface it stands in
 * for (paths are relative to the tile-rs source tree).
 */
#ifndef TILE_SM100_H_
#define TILE_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TSM100_VERSION 100 /* major*100 + minor */

/* ---- status codes ------------------------------------------------------- */
/* The reference reports failures as HalError variants
 * (crates/tile_hal/src/error.rs:5-35); each code names the variant a binding
 * should raise. */
enum {
  TSM100_OK = 0,
  TSM100_ERR_INVALID = 1,     /* bad argument / unsupported shape -> KernelError   */
  TSM100_ERR_NO_DEVICE = 2,   /* no CUDA device / driver          -> BackendNotAvailable */
  TSM100_ERR_MEMORY = 3,      /* allocation or copy failed        -> MemoryError   */
  TSM100_ERR_LAUNCH = 4,      /* kernel load or launch failed     -> KernelError   */
  TSM100_ERR_STREAM = 5,      /* stream / event failure           -> StreamError   */
  TSM100_ERR_RUNTIME = 6,     /* any other CUDA runtime error     -> RuntimeError  */
  TSM100_ERR_TIMEOUT = 7,     /* a bounded device-side wait ran out -> RuntimeError */
  TSM100_ERR_BUFFER = 8,      /* caller's output buffer too small (size returned) */
  TSM100_ERR_EMIT = 9         /* MLIR not accepted by the cuda_sm100 target -> Err(String) */
};

/* ---- element types ------------------------------------------------------ */
/* tile_hal's TileDtype (crates/tile_hal/src/kernel.rs:85-92) plus bf16, which
 * tile_std spells only as u16 bit patterns (crates/tile_std/src/tile.rs:2593-2601). */
enum {
  TSM100_F32 = 0,
  TSM100_F16 = 1,
  TSM100_BF16 = 2
};

typedef struct tsm100_device_s* tsm100_device_t; /* opaque */
typedef struct tsm100_module_s* tsm100_module_t; /* opaque */

/* ---- library / errors --------------------------------------------------- */
int32_t tsm100_version(void);
/* Copies the calling thread's last error message (NUL-terminated, truncated to
 * `cap`) and returns its full length.  Replaces the String carried by HalError
 * (crates/tile_hal/src/error.rs:5-35) and by CodegenTarget::emit's Err
 * (crates/tile_codegen/src/target.rs:64). */
size_t tsm100_last_error(char* buf, size_t cap);

/* ---- devices: crates/tile_hal/src/device.rs:25-57, cuda.rs:293-417 ------- */
/* cuDeviceGetCount (cuda.rs:330-337 `device_count`). */
int32_t tsm100_device_count(int32_t* count);
/* CudaDevice::new (cuda.rs:300-328): binds the device's primary context; any
 * number of devices may be open in one process, each call made with the right
 * device current (the reference creates one context and never re-selects it). */
int32_t tsm100_device_open(int32_t ordinal, tsm100_device_t* out);
int32_t tsm100_device_close(tsm100_device_t dev); /* Drop for CudaDevice, cuda.rs:411-417 */
int32_t tsm100_device_ordinal(tsm100_device_t dev, int32_t* ordinal); /* Device::ordinal */
int32_t tsm100_device_name(tsm100_device_t dev, char* buf, size_t cap); /* Device::name   */
/* Device::mem_info -> MemInfo{free,total} (device.rs:9-15, cuda.rs:373-380). */
int32_t tsm100_mem_info(tsm100_device_t dev, size_t* free_bytes, size_t* total_bytes);
/* Number of SMs; no counterpart in the reference (its grids are fixed by the emitter). */
int32_t tsm100_device_sm_count(tsm100_device_t dev, int32_t* sms);
/* Synchronises `stream`, then reads and clears the device's kernel status word:
 * 0, or 0x1000|site when a kernel gave up one of its bounded waits (mbarrier,
 * tensor-core completion).  The reference has no device-side error channel;
 * check_cu (crates/tile_hal/src/cuda.rs:124-130) sees driver codes only. */
int32_t tsm100_device_status(tsm100_device_t dev, void* stream, uint32_t* status);

/* Lets one bounded device-side wait run out on purpose: a one-CTA kernel waits up to
 * `limit_us` microseconds on a barrier nobody arrives at, gives up, records
 * 0x1000|63 in the device's status word and returns normally (no trap, no fault, no
 * unbounded spin).  The call itself returns TSM100_OK once that kernel has finished;
 * the next tsm100_stream_synchronize / tsm100_device_status on the device then
 * reports the timeout exactly as it would for a stuck pipeline, and clears it.
 * observed[0] = how many of the kernel's two waiting threads left through the failure
 * path (2), observed[1] = how long the first one waited, in microseconds.  May be
 * NULL.  No counterpart in the reference, which has no device-side error channel. */
int32_t tsm100_selftest_wait_timeout(tsm100_device_t dev, uint32_t limit_us, uint32_t* observed, void* stream);

/* ---- streams and events: crates/tile_hal/src/stream.rs:7-10, cuda.rs:134-166 */
/* A stream is a raw cudaStream_t carried as void*; NULL is the default stream,
 * so a stream made by another runtime in the same process can be passed. */
int32_t tsm100_stream_create(tsm100_device_t dev, void** stream);   /* Device::create_stream */
int32_t tsm100_stream_destroy(tsm100_device_t dev, void* stream);    /* Drop for CudaStream   */
int32_t tsm100_stream_synchronize(tsm100_device_t dev, void* stream); /* Stream::synchronize   */
/* 1 if all work on the stream has finished, 0 if not; the reference has no query. */
int32_t tsm100_stream_query(tsm100_device_t dev, void* stream, int32_t* done);
/* Events time kernels on the device; the reference HAL has no timing facility. */
int32_t tsm100_event_create(tsm100_device_t dev, void** event);
int32_t tsm100_event_record(tsm100_device_t dev, void* event, void* stream);
int32_t tsm100_event_synchronize(tsm100_device_t dev, void* event);
int32_t tsm100_event_elapsed_ms(tsm100_device_t dev, void* start, void* stop, float* ms);
int32_t tsm100_event_destroy(tsm100_device_t dev, void* event);

/* ---- buffers: crates/tile_hal/src/buffer.rs:32-55, cuda.rs:170-218, :339-371 */
int32_t tsm100_alloc(tsm100_device_t dev, size_t bytes, void** dptr); /* Device::alloc (cuMemAlloc) */
int32_t tsm100_free(tsm100_device_t dev, void* dptr);                  /* Drop for CudaBuffer        */
/* Page-locked host staging memory, so that copies can overlap kernels. */
int32_t tsm100_host_alloc(size_t bytes, void** hptr);
int32_t tsm100_host_free(void* hptr);
/* DeviceBuffer::copy_from_host / copy_to_host (cuda.rs:181-199).  Ordered on
 * `stream`; asynchronous with respect to the host when `host` is page-locked,
 * otherwise the call returns once the host buffer may be reused / is filled. */
int32_t tsm100_memcpy_h2d(tsm100_device_t dev, void* dst, const void* host, size_t bytes, void* stream);
int32_t tsm100_memcpy_d2h(tsm100_device_t dev, void* host, const void* src, size_t bytes, void* stream);
int32_t tsm100_memset(tsm100_device_t dev, void* dst, int32_t byte, size_t bytes, void* stream);

/* ---- kernel modules: crates/tile_hal/src/kernel.rs:23-42, cuda.rs:222-289 - */
/* KernelLauncher::load: `path` is a shared library built from the source
 * tsm100_emit() produced ("device object file or shared library",
 * kernel.rs:27-28). */
int32_t tsm100_module_load(tsm100_device_t dev, const char* path, tsm100_module_t* out);
int32_t tsm100_module_unload(tsm100_module_t mod);
/* KernelLauncher::launch(name, LaunchGrid, args, stream) (kernel.rs:35-41,
 * cuda.rs:245-288).  `blocks` is LaunchGrid::blocks = the number of per-block
 * tiles of the #[tile_kernel] contract (crates/tile_std_macros/src/lib.rs:237-254);
 * threads_per_block and shared_mem_bytes of LaunchGrid are chosen by the module
 * and therefore ignored.  `args` are the kernel's global-memory pointers in
 * declaration order. */
int32_t tsm100_launch(tsm100_module_t mod, const char* name, uint32_t blocks, void** args,
                      uint32_t nargs, void* stream);

/* ---- operators on device memory ---------------------------------------- */
/* Row softmax, y[r,:] = softmax(x[r,:]).  __tile_softmax_f32 / _f16
 * (crates/tile_std/src/tile.rs:189-190, :2162-2163; wrappers :2295-2305,
 * :2912-2920); semantics `linalg.softmax dimension(1)`
 * (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1305-1343).  Replaces the
 * lowering at crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1242-1336. */
typedef struct {
  int32_t dtype; /* TSM100_F32 | TSM100_F16 | TSM100_BF16 (storage; math is f32) */
  int64_t rows;
  int64_t cols;
} tsm100_softmax_desc;
int32_t tsm100_softmax(tsm100_device_t dev, const tsm100_softmax_desc* desc, const void* x, void* y,
                       void* stream);

/* RMS normalisation, y[r,c] = x[r,c] * rsqrt(mean_c(x[r,:]^2) + eps), no weight.
 * __tile_rms_norm_f32 (crates/tile_std/src/tile.rs:2063; wrapper :2731-2738);
 * semantics linalg.mul + linalg.reduce addf + rsqrt(sum / cols + eps) + multiply
 * (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1666-1767).  Replaces the lowering at
 * crates/rustc_codegen_tile/src/mlir_to_gpu.rs:920-977. */
typedef struct {
  int32_t dtype; /* storage type; math is f32 */
  int64_t rows;
  int64_t cols;
  float eps;
} tsm100_rms_norm_desc;
int32_t tsm100_rms_norm(tsm100_device_t dev, const tsm100_rms_norm_desc* desc, const void* x, void* y,
                        void* stream);

/* Row reduction to a ROWS x 1 tile, y[r] = sum_c x[r,c] or max_c x[r,c] (an empty row gives 0
 * or -inf).  __tile_reduce_sum_f32 / __tile_reduce_max_f32 (tile.rs:206-209; wrappers
 * :2352-2367); semantics linalg.fill + linalg.reduce (mlir_to_linalg.rs:545-550).  Replaces
 * the warp-only lowering at mlir_to_gpu.rs:2059-2092. */
#define TSM100_REDUCE_SUM 0
#define TSM100_REDUCE_MAX 1
typedef struct {
  int32_t dtype; /* storage type of x and y; accumulation is f32 */
  int32_t kind;  /* TSM100_REDUCE_SUM | TSM100_REDUCE_MAX */
  int64_t rows;
  int64_t cols;
} tsm100_reduce_desc;
int32_t tsm100_reduce(tsm100_device_t dev, const tsm100_reduce_desc* desc, const void* x, void* y,
                      void* stream);

/* y = silu(gate) * up element-wise, silu(x) = x / (1 + exp(-x)); up == NULL gives silu(gate).
 * __tile_silu_f32 / _f16 and __tile_mul_f32 / _f16 (tile.rs:229, :1135, :184, :2160; wrappers
 * :2416-2422, :2272-2282); semantics mlir_to_linalg.rs:774-782 and :425.  Replaces the fused
 * lowering at mlir_to_gpu.rs:542-641. */
typedef struct {
  int32_t dtype;
  int64_t rows;
  int64_t cols;
} tsm100_silu_mul_desc;
int32_t tsm100_silu_mul(tsm100_device_t dev, const tsm100_silu_mul_desc* desc, const void* gate,
                        const void* up, void* y, void* stream);

/* GEMM, C[M,N] = A[M,K] * B, all row-major, C overwritten (zero-initialised
 * accumulator).  __tile_matmul_f32 (tile.rs:192-193, :2307-2319),
 * __tile_matmul_f16 (tile.rs:1982-1986, :2593-2601, :2666-2674) and, with
 * b_transposed, __tile_matmul_transposed_* (tile.rs:2017-2031, :2682-2702;
 * B stored [N,K]); semantics linalg.fill 0 + linalg.matmul
 * (mlir_to_linalg.rs:1345-1393).  Replaces mlir_to_gpu.rs:1373-1397 (a TODO
 * comment) and :1584-1622.  16-bit inputs accumulate in f32 on the tensor
 * cores; out_dtype is the input dtype or TSM100_F32.  `batch` independent
 * problems are stored back to back (the per-block tile stride of
 * #[tile_kernel], tile_std_macros/src/lib.rs:237-254).
 * lda / ldb / ldc are row pitches in elements; 0 means "packed" (K for A; N, or K
 * when b_transposed, for B; N for C), which is the only layout the tile
 * intrinsics know.  A non-zero pitch lets a column block of a larger row-major
 * matrix be an operand or the result in place (the N-column split of one large
 * GEMM across GPUs); problems of a batch are then rows * pitch apart. */
typedef struct {
  int32_t dtype;     /* element type of A and B */
  int32_t out_dtype; /* element type of C */
  int32_t b_transposed;
  int32_t batch;
  int64_t m, n, k;
  int64_t lda, ldb, ldc; /* 0 = packed */
} tsm100_gemm_desc;
int32_t tsm100_gemm(tsm100_device_t dev, const tsm100_gemm_desc* desc, const void* a, const void* b,
                    void* c, void* stream);

/* The tensor-core GEMM of tsm100_gemm for callers that must not allocate device
 * memory; it has no counterpart in the reference.  It takes no device handle
 * (opening one allocates): it runs on the CUDA device that is current, and the one
 * word of scratch the kernel needs (where it reports a timed-out wait) lives in a
 * 256-byte static device array inside the library instead of in cudaMalloc'ed
 * memory.  Meant for code that runs while a CUDA graph is being captured elsewhere
 * in the process, for hosts that freeze the device heap after start-up, and for
 * loops that cannot afford cudaMalloc's implicit synchronisation.  It calls no
 * cudaMalloc, cudaFree or allocating library routine.
 *  - Only problems the tensor-core kernel takes are accepted (16-bit inputs,
 *    16-byte aligned pointers, K and, for row-major B, N multiples of 8, all
 *    dimensions positive); anything else, or a problem whose scratch need would
 *    exceed the 256 bytes, is TSM100_ERR_INVALID with a message.
 *  - The first call on each device looks the array's address up; make that call
 *    before any stream capture begins.
 *  - All calls share the array and it keeps the last call's contents; the entry
 *    point clears the word on `stream` before the kernel.  Two calls whose kernels
 *    overlap on the GPU (different streams) race on it.
 *  - status_host may be NULL; otherwise the status word (0, or 0x1000|site) is
 *    copied there on `stream` after the kernel — read it after synchronising. */
int32_t tsm100_gemm_static_scratch(const tsm100_gemm_desc* desc, const void* a, const void* b, void* c,
                                   void* stream, uint32_t* status_host);

/* Fused attention forward, O = softmax(Q K^T / sqrt(d)) V per (batch, head).
 * Q,O: [batch][heads_q][seq][head_dim]; K,V: [batch][heads_kv][seq][head_dim].
 * heads_q == heads_kv, causal = 0: __tile_attention_f32 (tile.rs:218-224,
 * :2389-2410; mlir_to_linalg.rs:1781-1902).  causal = 1 adds
 * __tile_causal_mask_f32 (tile.rs:1876-1877; mlir_to_linalg.rs:1191-1244)
 * between the scale and the softmax.  heads_q > heads_kv is
 * __tile_attention_gqa_* as the NVIDIA emitter defines it
 * (mlir_to_gpu.rs:1624-1711): kv_head = h / (heads_q/heads_kv), always causal
 * there.  Replaces mlir_to_gpu.rs:1976-1979 (unhandled) and :1624-1711.
 * 16-bit Q/K/V use tensor cores with f32 softmax statistics (head_dim 128: tcgen05; 32 / 64 / 96: warp-level
 * MMA); f32 Q/K/V with head_dim 32 / 64 / 96 / 128 use tensor cores with three TF32 products per product
 * (results agree with an f32 evaluation to 1e-5).  Other head sizes, or rows that do not start on 16-byte
 * boundaries: FP32 pipe. */
typedef struct {
  int32_t dtype; /* TSM100_BF16 | TSM100_F16 | TSM100_F32 */
  int32_t causal;
  int32_t batch;
  int32_t heads_q;
  int32_t heads_kv;
  int32_t seq;
  int32_t head_dim;
} tsm100_attention_desc;
int32_t tsm100_attention(tsm100_device_t dev, const tsm100_attention_desc* desc, const void* q,
                         const void* k, const void* v, void* o, void* stream);

/* ---- operators on HOST memory (upload, compute, download in one call) ---- */
/* Rotary position embedding, in place: the pair (x[2i], x[2i+1]) of every head of token s is rotated by
 * the angle (start_pos + s) * theta^(-2i / head_dim).  x is [batch][seq_len][heads][head_dim].
 * __tile_rope_inplace_f32 (seq_len 1, start_pos = the position) and __tile_rope_prefill_f32
 * (tile.rs:2113-2115, :2128-2129); arithmetic of crates/rustc_codegen_tile/src/mlir_to_msl.rs:10707-10728,
 * :10883-10908, whose run-time constants position / start_pos and theta are fields here. */
typedef struct {
  int32_t dtype;
  int32_t batch;
  int32_t seq_len;
  int32_t heads;
  int32_t head_dim; /* even */
  int32_t start_pos;
  float theta;
} tsm100_rope_desc;
int32_t tsm100_rope(tsm100_device_t dev, const tsm100_rope_desc* desc, void* x, void* stream);

/* KV-cache append: cache[b, h, start_pos + s, :] = src[b, s, h, :] with src [batch][seq_len][heads][head_dim]
 * and cache [batch][heads][max_seq][head_dim].  __tile_kv_cache_update_f32 (seq_len 1) and
 * __tile_kv_cache_update_prefill_f32 (tile.rs:2117-2119, :2131-2132; mlir_to_msl.rs:10730-10741, :10910-10926). */
typedef struct {
  int32_t dtype;
  int32_t batch;
  int32_t seq_len;
  int32_t heads;
  int32_t head_dim;
  int32_t start_pos;
  int32_t max_seq;
} tsm100_kv_cache_update_desc;
int32_t tsm100_kv_cache_update(tsm100_device_t dev, const tsm100_kv_cache_update_desc* desc, const void* src,
                               void* cache, void* stream);

/* Prefill attention: seq_len new tokens, already appended to the KV cache behind start_pos earlier ones, attend
 * causally: token s sees cache positions 0 .. start_pos + s.  q, o are token-major [seq_len][heads_q][head_dim],
 * the caches [heads_kv][max_seq][head_dim], kv head = h / (heads_q / heads_kv).
 * __tile_attention_prefill_f32 (tile.rs:2134-2136; wrapper :3062-3074); arithmetic of
 * crates/rustc_codegen_tile/src/mlir_to_msl.rs:10928-11010 without that lowering's limit of 256 cache positions
 * (its `threadgroup float scores[256]`).  The same kernels as tsm100_attention serve it (tensor cores for
 * head_dim 128 in 16 bit and for head_dim 32 / 64 / 96 / 128 in f32 and 32 / 64 / 96 in 16 bit). */
typedef struct {
  int32_t dtype;
  int32_t heads_q;
  int32_t heads_kv;
  int32_t seq_len;
  int32_t start_pos;
  int32_t max_seq;
  int32_t head_dim;
} tsm100_attention_prefill_desc;
int32_t tsm100_attention_prefill(tsm100_device_t dev, const tsm100_attention_prefill_desc* desc, const void* q,
                                 const void* k_cache, const void* v_cache, void* o, void* stream);

/* Single-token (decode) attention against a KV cache:
 *   o[b,h,:] = softmax_p(q[b,h,:] . K[b,g,p,:] / sqrt(d)) V[b,g,p,:],  p < seq_len,  g = h / (heads_q / heads_kv).
 * __tile_attention_decode_f32 (tile.rs:2120-2124; wrapper :3004-3018): q, o [heads_q][d], caches
 * [heads_kv][max_seq][d]; opaque in the linalg bridge (mlir_to_linalg.rs:502-505), arithmetic as the
 * five phases of the Metal lowering (crates/rustc_codegen_tile/src/mlir_to_msl.rs:10747-10812), whose
 * run-time constants seq_len, max_seq and the head counts are the fields below.  `batch` repeats the
 * problem: q, o [batch][heads_q][d], caches [batch][heads_kv][max_seq][d].  head_dim 64 or 128. */
typedef struct {
  int32_t dtype;    /* storage type of q, the caches and o; math is f32 */
  int32_t batch;
  int32_t heads_q;
  int32_t heads_kv;
  int32_t seq_len;  /* positions of the cache that are filled */
  int32_t max_seq;  /* row pitch of the cache, in positions */
  int32_t head_dim;
} tsm100_attention_decode_desc;
int32_t tsm100_attention_decode(tsm100_device_t dev, const tsm100_attention_decode_desc* desc, const void* q,
                                const void* k_cache, const void* v_cache, void* o, void* stream);

/* The path a tile_hal host program takes per kernel: alloc_from_slice ->
 * launch -> copy_to_host (crates/tile_hal/src/cuda.rs:348-371, :245-288,
 * :190-199), here chunked through page-locked staging so that copies in both
 * directions overlap the kernel.  Pointers are ordinary host memory.
 * tsm100_gemm_host keeps B resident and streams A and C in row blocks, each a
 * launch of its own: a 16-bit result may differ from tsm100_gemm on the whole
 * problem by one rounding of the stored type in a few elements (the f32 sums
 * are taken in another order); f32 results do not differ. */
int32_t tsm100_softmax_host(tsm100_device_t dev, const tsm100_softmax_desc* desc, const void* x,
                            void* y);
int32_t tsm100_gemm_host(tsm100_device_t dev, const tsm100_gemm_desc* desc, const void* a,
                         const void* b, void* c);
int32_t tsm100_attention_host(tsm100_device_t dev, const tsm100_attention_desc* desc, const void* q,
                              const void* k, const void* v, void* o);

/* ---- sharding across GPUs ---------------------------------------------- */
/* Splits `units` independent work units (softmax rows, GEMM batches or
 * N-column blocks, attention (batch, kv-head) groups) over `world` ranks in
 * contiguous blocks; the first units % world ranks get one more.  The reference
 * is single-device (crates/tile_hal/src/backend.rs:95-112); the unit is the
 * per-block tile of #[tile_kernel] (tile_std_macros/src/lib.rs:237-254). */
int32_t tsm100_shard_range(int64_t units, int32_t world, int32_t rank, int64_t* first, int64_t* count);

/* ---- multi-GPU launcher --------------------------------------------------- */
/* One problem, described once with HOST buffers, run on a list of devices of this
 * machine.  The reference can drive one GPU per process (crates/tile_hal/src/cuda.rs:321-327:
 * one cuCtxCreate, no cuCtxSetCurrent; crates/tile_hal/src/backend.rs:95-112); the path has
 * no exchange step, so the launcher deals the problem's independent units out with
 * tsm100_shard_range and gives every device a host thread, a stream and a workspace of its
 * own.  No peer access, no collective.  Units: softmax rows; GEMM problems of a batch, or,
 * for batch == 1, N columns in blocks of 256 (device g computes C[:, first:first+count) from
 * all of A and its columns of B, read from and written into the caller's row-major matrices
 * in place); attention (batch, KV head) groups. */
enum { TSM100_OP_SOFTMAX = 0, TSM100_OP_GEMM = 1, TSM100_OP_ATTENTION = 2 };
typedef struct {
  int32_t op;         /* TSM100_OP_* */
  const void* desc;   /* tsm100_softmax_desc | tsm100_gemm_desc | tsm100_attention_desc of the WHOLE problem */
  const void* in[3];  /* host buffers: x | a, b | q, k, v (page-locked ones copy asynchronously) */
  void* out;          /* host buffer:  y | c | o */
  int32_t launches;   /* kernel launches per device on its resident shard, timed together (< 1 means 1) */
  int32_t timeout_ms; /* limit for each device's whole part; 0 = none */
} tsm100_multi_job;
typedef struct {
  int32_t ordinal;
  int32_t status;         /* TSM100_* of this device's part */
  int64_t first, count;   /* its shard, in units */
  float upload_ms;        /* CUDA-event times on the device's stream ... */
  float kernel_ms;        /* ... per launch */
  float download_ms;
  float total_ms;         /* host clock around everything the device's thread did */
  uint32_t device_status; /* the kernels' status word (0, or 0x1000|site) */
  char message[160];      /* names the device when status != TSM100_OK */
} tsm100_multi_report;
/* The shard device `index` of `n` gets: contiguous, whole granules, the first ones one larger. */
int32_t tsm100_multi_plan(const tsm100_multi_job* job, int32_t n, int32_t index, int64_t* first, int64_t* count);
/* Runs the job on devices ordinals[0..n) and fills reports[0..n).  Returns TSM100_OK, or the
 * status of the first device that failed, with a message that names its ordinal.  A device
 * past timeout_ms is reported as TSM100_ERR_TIMEOUT; the call still returns only after that
 * device has drained, because its copies target the caller's buffers (every device-side wait
 * of the kernels is itself bounded, so it does drain).  Device workspaces are kept between
 * runs; tsm100_multi_release frees them. */
int32_t tsm100_multi_run(const tsm100_multi_job* job, const int32_t* ordinals, int32_t n, tsm100_multi_report* reports);
/* The same scheduling (split, one thread per device, clock watching, reports) around a
 * caller-supplied per-device function; NULL selects the built-in CUDA one.  This is how
 * the launcher's failure handling is tested on machines without GPUs. */
typedef int32_t (*tsm100_multi_worker_fn)(void* user, const tsm100_multi_job* job, int32_t ordinal, int64_t first,
                                          int64_t count, tsm100_multi_report* report);
int32_t tsm100_multi_run_with(const tsm100_multi_job* job, const int32_t* ordinals, int32_t n,
                              tsm100_multi_report* reports, tsm100_multi_worker_fn worker, void* user);
int32_t tsm100_multi_release(void);

/* ---- cuda_sm100 CodegenTarget ------------------------------------------ */
/* CodegenTarget::emit for the target named "cuda_sm100"
 * (crates/tile_codegen/src/target.rs:57-65; supersedes convert_mlir_to_gpu,
 * crates/rustc_codegen_tile/src/mlir_to_gpu.rs:62-99).  Pure and deterministic:
 * reads `mlir` only.  Writes the CUDA translation unit (EmitOut.source, ext
 * "cu") to `source`, and the entry kernel names (TargetMeta.kernel_names,
 * target.rs:33-38) to `names`, separated by '\n'.  *source_len / *names_len
 * receive the full lengths (without NUL); TSM100_ERR_BUFFER if a buffer is too
 * small (call again with larger ones).  TSM100_ERR_EMIT for an empty module, a
 * module with no `hacc.entry` kernel, or an intrinsic outside the target's
 * scope — never a silent TODO comment. */
int32_t tsm100_emit(const char* mlir, size_t mlir_len, char* source, size_t source_cap,
                    size_t* source_len, char* names, size_t names_cap, size_t* names_len);
/* The TileKernel descriptors of the module's entry kernels ("the compiler emits a TileKernel
 * descriptor alongside the compiled binary", crates/tile_hal/src/kernel.rs:160-181; TileOp
 * :93-158), as a JSON array with one object per kernel in the order of tsm100_emit's names:
 *   {"name", "mode": "Vector" | "General" (TileKernel::inferred_mode, kernel.rs:204-211),
 *    "num_inputs", "num_outputs", "ops": [{"op": "<TileOp variant>", <its fields>} ...],
 *    "args": [{"index", "role": "input" | "output" | "unused", "dtype", "elements_per_block"} ...]}
 * "args" is what a launcher needs to validate buffer sizes for a LaunchGrid (blocks *
 * elements_per_block elements of dtype).  Same purity and error behaviour as tsm100_emit. */
int32_t tsm100_emit_descriptors(const char* mlir, size_t mlir_len, char* json, size_t json_cap,
                                size_t* json_len);
const char* tsm100_target_name(void); /* CodegenTarget::name -> "cuda_sm100" */
const char* tsm100_target_ext(void);  /* EmitOut.ext        -> "cu"         */

/* ---- seeded synthetic inputs (host) ------------------------------------- */
/* Counter-based generator shared by tests and benchmarks, so that the GPU and
 * the CPU oracle read identical host buffers.  Element i of a stream with seed
 * s is a function of (s, i) only.  No counterpart in the reference.
 *   uniform: [-1, 1) from the top 24 bits of SplitMix64(s ^ i*0x9E3779B97F4A7C15)
 *   normal : Box-Muller in f64 on the index pair (2p, 2p+1), times sigma
 *   outliers: element i := value where SplitMix64(s ^ i*golden) % period == 0 */
int32_t tsm100_fill_uniform_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index);
int32_t tsm100_fill_normal_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index, double sigma);
/* The normal stream of tsm100_fill_normal_f32, times `factor` in f32, rounded to bf16 (RNE): the same bits as
 * fill + scale + f32_to_bf16 without the f32 buffer. */
int32_t tsm100_fill_normal_bf16(uint16_t* dst, int64_t n, uint64_t seed, int64_t first_index, double sigma, float factor);
int32_t tsm100_plant_outliers_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index,
                                  uint32_t period, float value);
int32_t tsm100_scale_f32(float* dst, int64_t n, float factor);
int32_t tsm100_f32_to_bf16(const float* src, uint16_t* dst, int64_t n); /* arith.truncf, RNE */
int32_t tsm100_bf16_to_f32(const uint16_t* src, float* dst, int64_t n); /* arith.extf */

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* TILE_SM100_H_ */
