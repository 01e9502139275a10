//! `tile_hal` and `tile_codegen` implementations over `libtile_sm100`.  Forwarding code only; not compiled
//! in the image this library was developed in (no Rust toolchain there).
//!
//! Trait definitions followed: `crates/tile_hal/src/device.rs:25-57`, `stream.rs:7-10`, `buffer.rs:32-55`,
//! `kernel.rs:23-42`, `error.rs:5-35`, `backend.rs:118-125`; `crates/tile_codegen/src/target.rs:17-65`.
use std::ffi::{c_void, CString};
use std::marker::PhantomData;
use std::path::Path;
use std::sync::Arc;

use tile_codegen::{CodegenTarget, EmitOpts, EmitOut, TargetMeta};
use tile_hal::{Device, DeviceBuffer, DeviceRepr, HalError, HalResult, KernelLauncher, KernelMode, LaunchGrid, MemInfo, Stream};
use tile_sm100_sys as sys;

/// Status code -> the `HalError` variant the header names for it.
fn check(status: i32) -> HalResult<()> {
    let msg = || sys::last_error();
    match status {
        sys::OK => Ok(()),
        sys::ERR_INVALID | sys::ERR_LAUNCH | sys::ERR_EMIT => Err(HalError::KernelError(msg())),
        sys::ERR_NO_DEVICE => Err(HalError::BackendNotAvailable(msg())),
        sys::ERR_MEMORY => Err(HalError::MemoryError(msg())),
        sys::ERR_STREAM => Err(HalError::StreamError(msg())),
        _ => Err(HalError::RuntimeError(msg())), // ERR_RUNTIME, ERR_TIMEOUT, ERR_BUFFER
    }
}

/// Owns the `tsm100_device_t`; shared by everything created from the device so that handles stay valid.
struct Handle(sys::Device);
unsafe impl Send for Handle {}
unsafe impl Sync for Handle {}
impl Drop for Handle {
    fn drop(&mut self) {
        unsafe { sys::tsm100_device_close(self.0) };
    }
}

pub struct Sm100Device {
    handle: Arc<Handle>,
    ordinal: u32,
    name: String,
}

impl Sm100Device {
    /// `CudaDevice::new` (`crates/tile_hal/src/cuda.rs:300-328`); any number of devices may be open at once.
    pub fn new(ordinal: u32) -> HalResult<Self> {
        let mut dev: sys::Device = std::ptr::null_mut();
        check(unsafe { sys::tsm100_device_open(ordinal as i32, &mut dev) })?;
        let handle = Arc::new(Handle(dev));
        let mut buf = vec![0u8; 256];
        check(unsafe { sys::tsm100_device_name(dev, buf.as_mut_ptr() as *mut _, buf.len()) })?;
        let end = buf.iter().position(|&b| b == 0).unwrap_or(buf.len());
        Ok(Self { handle, ordinal, name: String::from_utf8_lossy(&buf[..end]).into_owned() })
    }
    pub fn device_count() -> HalResult<u32> {
        let mut n = 0i32;
        check(unsafe { sys::tsm100_device_count(&mut n) })?;
        Ok(n as u32)
    }
    pub fn raw(&self) -> sys::Device {
        self.handle.0
    }
}

pub struct Sm100Stream {
    handle: Arc<Handle>,
    raw: sys::RawStream,
}
unsafe impl Send for Sm100Stream {}
impl Sm100Stream {
    pub fn raw(&self) -> sys::RawStream {
        self.raw
    }
}
impl Stream for Sm100Stream {
    /// Also surfaces a kernel that gave up one of its bounded device-side waits (TSM100_ERR_TIMEOUT -> RuntimeError).
    fn synchronize(&self) -> HalResult<()> {
        check(unsafe { sys::tsm100_stream_synchronize(self.handle.0, self.raw) })
    }
}
impl Drop for Sm100Stream {
    fn drop(&mut self) {
        unsafe { sys::tsm100_stream_destroy(self.handle.0, self.raw) };
    }
}

pub struct Sm100Buffer<T: DeviceRepr> {
    handle: Arc<Handle>,
    ptr: *mut c_void,
    len: usize,
    _t: PhantomData<T>,
}
unsafe impl<T: DeviceRepr> Send for Sm100Buffer<T> {}
impl<T: DeviceRepr> DeviceBuffer<T> for Sm100Buffer<T> {
    fn len(&self) -> usize {
        self.len
    }
    /// The copy is ordered on the default stream and the call returns once the slice may be reused; the trait's
    /// `&dyn Stream` cannot be downcast, so, like the reference's backend (`cuda.rs:181-188`), it is only synchronised.
    fn copy_from_host(&mut self, src: &[T], stream: &dyn Stream) -> HalResult<()> {
        if src.len() != self.len {
            return Err(HalError::MemoryError(format!("copy_from_host: {} elements into a buffer of {}", src.len(), self.len)));
        }
        check(unsafe { sys::tsm100_memcpy_h2d(self.handle.0, self.ptr, src.as_ptr() as *const c_void, std::mem::size_of_val(src), std::ptr::null_mut()) })?;
        check(unsafe { sys::tsm100_stream_synchronize(self.handle.0, std::ptr::null_mut()) })?;
        stream.synchronize()
    }
    fn copy_to_host(&self, stream: &dyn Stream) -> HalResult<Vec<T>> {
        stream.synchronize()?; // the kernels that produced the data
        let mut out = Vec::<T>::with_capacity(self.len);
        check(unsafe { sys::tsm100_memcpy_d2h(self.handle.0, out.as_mut_ptr() as *mut c_void, self.ptr, self.len * std::mem::size_of::<T>(), std::ptr::null_mut()) })?;
        check(unsafe { sys::tsm100_stream_synchronize(self.handle.0, std::ptr::null_mut()) })?;
        unsafe { out.set_len(self.len) };
        Ok(out)
    }
    fn as_raw_ptr(&self) -> *const c_void {
        self.ptr
    }
    fn as_raw_mut_ptr(&mut self) -> *mut c_void {
        self.ptr
    }
}
impl<T: DeviceRepr> Drop for Sm100Buffer<T> {
    fn drop(&mut self) {
        unsafe { sys::tsm100_free(self.handle.0, self.ptr) };
    }
}

pub struct Sm100Launcher {
    handle: Arc<Handle>,
    modules: Vec<sys::Module>,
}
unsafe impl Send for Sm100Launcher {}
impl KernelLauncher for Sm100Launcher {
    type Stream = Sm100Stream;
    /// `path` is the shared library nvcc built from `EmitOut.source` ("device object file or shared library",
    /// `kernel.rs:27-28`).  `mode` is a property of the emitted module and is ignored.
    fn load(&mut self, path: &Path, _mode: KernelMode) -> HalResult<()> {
        let c = CString::new(path.to_string_lossy().as_bytes()).map_err(|e| HalError::KernelError(e.to_string()))?;
        let mut m: sys::Module = std::ptr::null_mut();
        check(unsafe { sys::tsm100_module_load(self.handle.0, c.as_ptr(), &mut m) })?;
        self.modules.push(m);
        Ok(())
    }
    /// `grid.blocks` = the number of per-block tiles of the `#[tile_kernel]` contract; threads and shared memory are
    /// the module's business.  The kernel is looked up in the modules in load order.
    unsafe fn launch(&self, name: &str, grid: LaunchGrid, args: &mut [*mut c_void], stream: &Self::Stream) -> HalResult<()> {
        let c = CString::new(name).map_err(|e| HalError::KernelError(e.to_string()))?;
        let mut last = HalError::KernelError(format!("no module loaded; cannot launch {name}"));
        for &m in &self.modules {
            match check(sys::tsm100_launch(m, c.as_ptr(), grid.blocks, args.as_mut_ptr(), args.len() as u32, stream.raw())) {
                Ok(()) => return Ok(()),
                Err(e) => last = e,
            }
        }
        Err(last)
    }
}
impl Drop for Sm100Launcher {
    fn drop(&mut self) {
        for &m in &self.modules {
            unsafe { sys::tsm100_module_unload(m) };
        }
    }
}

impl Device for Sm100Device {
    type Stream = Sm100Stream;
    type Buffer<T: DeviceRepr> = Sm100Buffer<T>;
    type Launcher = Sm100Launcher;
    fn ordinal(&self) -> u32 {
        self.ordinal
    }
    fn name(&self) -> &str {
        &self.name
    }
    fn create_stream(&self) -> HalResult<Self::Stream> {
        let mut s: sys::RawStream = std::ptr::null_mut();
        check(unsafe { sys::tsm100_stream_create(self.raw(), &mut s) })?;
        Ok(Sm100Stream { handle: self.handle.clone(), raw: s })
    }
    fn alloc<T: DeviceRepr>(&self, count: usize) -> HalResult<Self::Buffer<T>> {
        let mut p: *mut c_void = std::ptr::null_mut();
        check(unsafe { sys::tsm100_alloc(self.raw(), count * std::mem::size_of::<T>(), &mut p) })?;
        Ok(Sm100Buffer { handle: self.handle.clone(), ptr: p, len: count, _t: PhantomData })
    }
    fn alloc_from_slice<T: DeviceRepr>(&self, data: &[T], stream: &Self::Stream) -> HalResult<Self::Buffer<T>> {
        let buf = self.alloc::<T>(data.len())?;
        check(unsafe { sys::tsm100_memcpy_h2d(self.raw(), buf.ptr, data.as_ptr() as *const c_void, std::mem::size_of_val(data), stream.raw()) })?;
        stream.synchronize()?; // the slice is pageable memory the caller may drop
        Ok(buf)
    }
    fn mem_info(&self) -> HalResult<MemInfo> {
        let (mut free, mut total) = (0usize, 0usize);
        check(unsafe { sys::tsm100_mem_info(self.raw(), &mut free, &mut total) })?;
        Ok(MemInfo { free, total })
    }
    fn create_launcher(&self) -> HalResult<Self::Launcher> {
        Ok(Sm100Launcher { handle: self.handle.clone(), modules: Vec::new() })
    }
}

/// The `cuda_sm100` target.  Registered with `registry.register(Box::new(CudaSm100Target))` next to
/// `crates/tile_codegen/src/targets.rs:62`, before the built-in "gpu" target if it is to shadow it.
pub struct CudaSm100Target;
impl CodegenTarget for CudaSm100Target {
    fn name(&self) -> &'static str {
        "cuda_sm100"
    }
    /// Pure and deterministic: reads `mlir_text` only (`target.rs:62-64`).  `opts.hw` describes Ascend's unified
    /// buffer and is ignored, as every host-toolchain target does.
    fn emit(&self, mlir_text: &str, _opts: &EmitOpts) -> Result<EmitOut, String> {
        let (mut src, mut names) = (vec![0u8; 2 * mlir_text.len() + 8192], vec![0u8; 4096]);
        let (mut sl, mut nl) = (0usize, 0usize);
        loop {
            let st = unsafe {
                sys::tsm100_emit(mlir_text.as_ptr() as *const _, mlir_text.len(), src.as_mut_ptr() as *mut _, src.len(), &mut sl,
                                 names.as_mut_ptr() as *mut _, names.len(), &mut nl)
            };
            match st {
                sys::OK => break,
                sys::ERR_BUFFER => {
                    src.resize(sl + 1, 0);
                    names.resize(nl + 1, 0);
                }
                _ => return Err(sys::last_error()),
            }
        }
        Ok(EmitOut {
            source: String::from_utf8_lossy(&src[..sl]).into_owned(),
            ext: "cu",
            meta: TargetMeta {
                has_cube_kernel: false,
                kernel_names: String::from_utf8_lossy(&names[..nl]).lines().map(str::to_owned).collect(),
            },
        })
    }
}

/// One problem on several GPUs (`tsm100_multi_run`): host buffers in, host buffers out, one report per device.
pub fn multi_run(job: &sys::MultiJob, ordinals: &[i32]) -> HalResult<Vec<sys::MultiReport>> {
    let mut reports: Vec<sys::MultiReport> = Vec::with_capacity(ordinals.len());
    let st = unsafe { sys::tsm100_multi_run(job, ordinals.as_ptr(), ordinals.len() as i32, reports.as_mut_ptr()) };
    unsafe { reports.set_len(ordinals.len()) };
    check(st).map(|_| reports)
}
