//! `extern "C"` declarations of `include/tile_sm100.h`, one for one.  Not compiled in the image this
//! library was developed in (no Rust toolchain there); the layout of every `#[repr(C)]` struct is the
//! header's, field for field.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_void};

pub const OK: i32 = 0;
pub const ERR_INVALID: i32 = 1;
pub const ERR_NO_DEVICE: i32 = 2;
pub const ERR_MEMORY: i32 = 3;
pub const ERR_LAUNCH: i32 = 4;
pub const ERR_STREAM: i32 = 5;
pub const ERR_RUNTIME: i32 = 6;
pub const ERR_TIMEOUT: i32 = 7;
pub const ERR_BUFFER: i32 = 8;
pub const ERR_EMIT: i32 = 9;
pub const F32: i32 = 0;
pub const F16: i32 = 1;
pub const BF16: i32 = 2;
pub const OP_SOFTMAX: i32 = 0;
pub const OP_GEMM: i32 = 1;
pub const OP_ATTENTION: i32 = 2;

pub type Device = *mut c_void;
pub type Module = *mut c_void;
pub type RawStream = *mut c_void; // cudaStream_t; null = the default stream
pub type RawEvent = *mut c_void;

#[repr(C)] #[derive(Clone, Copy, Default)] pub struct SoftmaxDesc { pub dtype: i32, pub rows: i64, pub cols: i64 }
#[repr(C)] #[derive(Clone, Copy, Default)] pub struct RmsNormDesc { pub dtype: i32, pub rows: i64, pub cols: i64, pub eps: f32 }
#[repr(C)] #[derive(Clone, Copy, Default)] pub struct ReduceDesc { pub dtype: i32, pub kind: i32, pub rows: i64, pub cols: i64 }
#[repr(C)] #[derive(Clone, Copy, Default)] pub struct SiluMulDesc { pub dtype: i32, pub rows: i64, pub cols: i64 }
/// lda / ldb / ldc: row pitches in elements, 0 = packed.
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct GemmDesc { pub dtype: i32, pub out_dtype: i32, pub b_transposed: i32, pub batch: i32, pub m: i64, pub n: i64, pub k: i64,
                      pub lda: i64, pub ldb: i64, pub ldc: i64 }
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct AttentionDesc { pub dtype: i32, pub causal: i32, pub batch: i32, pub heads_q: i32, pub heads_kv: i32, pub seq: i32, pub head_dim: i32 }
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct RopeDesc { pub dtype: i32, pub batch: i32, pub seq_len: i32, pub heads: i32, pub head_dim: i32, pub start_pos: i32, pub theta: f32 }
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct KvCacheUpdateDesc { pub dtype: i32, pub batch: i32, pub seq_len: i32, pub heads: i32, pub head_dim: i32, pub start_pos: i32, pub max_seq: i32 }
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct AttentionPrefillDesc { pub dtype: i32, pub heads_q: i32, pub heads_kv: i32, pub seq_len: i32, pub start_pos: i32, pub max_seq: i32, pub head_dim: i32 }
#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct AttentionDecodeDesc { pub dtype: i32, pub batch: i32, pub heads_q: i32, pub heads_kv: i32, pub seq_len: i32, pub max_seq: i32, pub head_dim: i32 }
#[repr(C)] #[derive(Clone, Copy)]
pub struct MultiJob { pub op: i32, pub desc: *const c_void, pub inputs: [*const c_void; 3], pub out: *mut c_void, pub launches: i32, pub timeout_ms: i32 }
#[repr(C)] #[derive(Clone, Copy)]
pub struct MultiReport { pub ordinal: i32, pub status: i32, pub first: i64, pub count: i64, pub upload_ms: f32, pub kernel_ms: f32,
                         pub download_ms: f32, pub total_ms: f32, pub device_status: u32, pub message: [c_char; 160] }
pub type MultiWorkerFn = Option<unsafe extern "C" fn(user: *mut c_void, job: *const MultiJob, ordinal: i32, first: i64, count: i64,
                                                     report: *mut MultiReport) -> i32>;

extern "C" {
    // library / errors
    pub fn tsm100_version() -> i32;
    pub fn tsm100_last_error(buf: *mut c_char, cap: usize) -> usize;
    // devices
    pub fn tsm100_device_count(count: *mut i32) -> i32;
    pub fn tsm100_device_open(ordinal: i32, out: *mut Device) -> i32;
    pub fn tsm100_device_close(dev: Device) -> i32;
    pub fn tsm100_device_ordinal(dev: Device, ordinal: *mut i32) -> i32;
    pub fn tsm100_device_name(dev: Device, buf: *mut c_char, cap: usize) -> i32;
    pub fn tsm100_mem_info(dev: Device, free: *mut usize, total: *mut usize) -> i32;
    pub fn tsm100_device_sm_count(dev: Device, sms: *mut i32) -> i32;
    pub fn tsm100_device_status(dev: Device, stream: RawStream, status: *mut u32) -> i32;
    pub fn tsm100_selftest_wait_timeout(dev: Device, limit_us: u32, observed: *mut u32, stream: RawStream) -> i32;
    // streams and events
    pub fn tsm100_stream_create(dev: Device, stream: *mut RawStream) -> i32;
    pub fn tsm100_stream_destroy(dev: Device, stream: RawStream) -> i32;
    pub fn tsm100_stream_synchronize(dev: Device, stream: RawStream) -> i32;
    pub fn tsm100_stream_query(dev: Device, stream: RawStream, done: *mut i32) -> i32;
    pub fn tsm100_event_create(dev: Device, event: *mut RawEvent) -> i32;
    pub fn tsm100_event_record(dev: Device, event: RawEvent, stream: RawStream) -> i32;
    pub fn tsm100_event_synchronize(dev: Device, event: RawEvent) -> i32;
    pub fn tsm100_event_elapsed_ms(dev: Device, start: RawEvent, stop: RawEvent, ms: *mut f32) -> i32;
    pub fn tsm100_event_destroy(dev: Device, event: RawEvent) -> i32;
    // buffers
    pub fn tsm100_alloc(dev: Device, bytes: usize, dptr: *mut *mut c_void) -> i32;
    pub fn tsm100_free(dev: Device, dptr: *mut c_void) -> i32;
    pub fn tsm100_host_alloc(bytes: usize, hptr: *mut *mut c_void) -> i32;
    pub fn tsm100_host_free(hptr: *mut c_void) -> i32;
    pub fn tsm100_memcpy_h2d(dev: Device, dst: *mut c_void, host: *const c_void, bytes: usize, stream: RawStream) -> i32;
    pub fn tsm100_memcpy_d2h(dev: Device, host: *mut c_void, src: *const c_void, bytes: usize, stream: RawStream) -> i32;
    pub fn tsm100_memset(dev: Device, dst: *mut c_void, byte: i32, bytes: usize, stream: RawStream) -> i32;
    // kernel modules
    pub fn tsm100_module_load(dev: Device, path: *const c_char, out: *mut Module) -> i32;
    pub fn tsm100_module_unload(module: Module) -> i32;
    pub fn tsm100_launch(module: Module, name: *const c_char, blocks: u32, args: *mut *mut c_void, nargs: u32, stream: RawStream) -> i32;
    // operators on device memory
    pub fn tsm100_softmax(dev: Device, d: *const SoftmaxDesc, x: *const c_void, y: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_rms_norm(dev: Device, d: *const RmsNormDesc, x: *const c_void, y: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_reduce(dev: Device, d: *const ReduceDesc, x: *const c_void, y: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_silu_mul(dev: Device, d: *const SiluMulDesc, gate: *const c_void, up: *const c_void, y: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_gemm(dev: Device, d: *const GemmDesc, a: *const c_void, b: *const c_void, c: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_gemm_static_scratch(d: *const GemmDesc, a: *const c_void, b: *const c_void, c: *mut c_void, stream: RawStream,
                                      status_host: *mut u32) -> i32;
    pub fn tsm100_attention(dev: Device, d: *const AttentionDesc, q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void,
                            stream: RawStream) -> i32;
    pub fn tsm100_rope(dev: Device, d: *const RopeDesc, x: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_kv_cache_update(dev: Device, d: *const KvCacheUpdateDesc, src: *const c_void, cache: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_attention_prefill(dev: Device, d: *const AttentionPrefillDesc, q: *const c_void, k_cache: *const c_void,
                                    v_cache: *const c_void, o: *mut c_void, stream: RawStream) -> i32;
    pub fn tsm100_attention_decode(dev: Device, d: *const AttentionDecodeDesc, q: *const c_void, k_cache: *const c_void,
                                   v_cache: *const c_void, o: *mut c_void, stream: RawStream) -> i32;
    // operators on host memory
    pub fn tsm100_softmax_host(dev: Device, d: *const SoftmaxDesc, x: *const c_void, y: *mut c_void) -> i32;
    pub fn tsm100_gemm_host(dev: Device, d: *const GemmDesc, a: *const c_void, b: *const c_void, c: *mut c_void) -> i32;
    pub fn tsm100_attention_host(dev: Device, d: *const AttentionDesc, q: *const c_void, k: *const c_void, v: *const c_void, o: *mut c_void) -> i32;
    // sharding and the multi-GPU launcher
    pub fn tsm100_shard_range(units: i64, world: i32, rank: i32, first: *mut i64, count: *mut i64) -> i32;
    pub fn tsm100_multi_plan(job: *const MultiJob, n: i32, index: i32, first: *mut i64, count: *mut i64) -> i32;
    pub fn tsm100_multi_run(job: *const MultiJob, ordinals: *const i32, n: i32, reports: *mut MultiReport) -> i32;
    pub fn tsm100_multi_run_with(job: *const MultiJob, ordinals: *const i32, n: i32, reports: *mut MultiReport, worker: MultiWorkerFn,
                                 user: *mut c_void) -> i32;
    pub fn tsm100_multi_release() -> i32;
    // the cuda_sm100 CodegenTarget
    pub fn tsm100_emit(mlir: *const c_char, len: usize, src: *mut c_char, src_cap: usize, src_len: *mut usize, names: *mut c_char,
                       names_cap: usize, names_len: *mut usize) -> i32;
    pub fn tsm100_emit_descriptors(mlir: *const c_char, len: usize, json: *mut c_char, cap: usize, json_len: *mut usize) -> i32;
    pub fn tsm100_target_name() -> *const c_char;
    pub fn tsm100_target_ext() -> *const c_char;
    // seeded synthetic inputs
    pub fn tsm100_fill_uniform_f32(dst: *mut f32, n: i64, seed: u64, first_index: i64) -> i32;
    pub fn tsm100_fill_normal_f32(dst: *mut f32, n: i64, seed: u64, first_index: i64, sigma: f64) -> i32;
    pub fn tsm100_fill_normal_bf16(dst: *mut u16, n: i64, seed: u64, first_index: i64, sigma: f64, factor: f32) -> i32;
    pub fn tsm100_plant_outliers_f32(dst: *mut f32, n: i64, seed: u64, first_index: i64, period: u32, value: f32) -> i32;
    pub fn tsm100_scale_f32(dst: *mut f32, n: i64, factor: f32) -> i32;
    pub fn tsm100_f32_to_bf16(src: *const f32, dst: *mut u16, n: i64) -> i32;
    pub fn tsm100_bf16_to_f32(src: *const u16, dst: *mut f32, n: i64) -> i32;
}

/// The calling thread's last error message (`tsm100_last_error`).
pub fn last_error() -> String {
    let mut buf = vec![0u8; 1024];
    let n = unsafe { tsm100_last_error(buf.as_mut_ptr() as *mut c_char, buf.len()) };
    buf.truncate(n.min(buf.len() - 1));
    String::from_utf8_lossy(&buf).into_owned()
}
