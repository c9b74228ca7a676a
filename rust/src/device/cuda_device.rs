//! CUDA device: the counterpart of `MetalDevice` (src/device/metal_device.rs) over the C ABI
//! of libtlcuda.  UNCOMPILED in this repository (no Rust toolchain in the build image).
//!
//! One `tlc_ctx` per GPU per host thread; calls on a context are ordered on its stream,
//! which matches the single-threaded interpreter (`&mut self` everywhere upstream).

use std::ffi::{CStr, CString};
use std::sync::Arc;

use crate::device::cuda_ffi as ffi;
use crate::error::{TensorError, TensorResult};

/// Turns a libtlcuda status into the `TensorError` variant it is numbered after
/// (src/error.rs:9-49); the message is the library's thread-local last error.
pub fn check(status: i32) -> TensorResult<()> {
    if status == ffi::TLC_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::tlc_last_error()) }.to_string_lossy().into_owned();
    Err(match status {
        ffi::TLC_ERR_SHAPE_MISMATCH => TensorError::InvalidOperation(msg), // ShapeMismatch carries two shapes upstream
        ffi::TLC_ERR_INVALID_OPERATION => TensorError::InvalidOperation(msg),
        ffi::TLC_ERR_DEVICE => TensorError::DeviceConversionError(msg),
        ffi::TLC_ERR_CUDA => TensorError::MetalError(msg),
        ffi::TLC_ERR_ALLOCATION => TensorError::AllocationError(msg),
        ffi::TLC_ERR_LOAD => TensorError::LoadError(msg),
        ffi::TLC_ERR_BUFFER_EXHAUSTED => TensorError::BufferExhausted(msg),
        ffi::TLC_ERR_INDEX => TensorError::InvalidOperation(msg),
        ffi::TLC_ERR_INVALID_DIMENSION => TensorError::InvalidOperation(msg),
        _ => TensorError::MetalError(msg), // TLC_ERR_TIMEOUT, TLC_ERR_COMM: device-side failures
    })
}

struct CtxHandle(*mut ffi::TlcCtx);
// The context is only used from the interpreter's thread; the handle travels inside Arc.
unsafe impl Send for CtxHandle {}
unsafe impl Sync for CtxHandle {}
impl Drop for CtxHandle {
    fn drop(&mut self) {
        unsafe { ffi::tlc_destroy(self.0) };
    }
}

/// `MetalDevice::new()` is a process-wide singleton behind `OnceLock`
/// (metal_device.rs:10, :36-45); so is `CudaDevice::new()`.
#[derive(Clone)]
pub struct CudaDevice {
    ctx: Arc<CtxHandle>,
    ordinal: i32,
}

static DEVICE: std::sync::OnceLock<CudaDevice> = std::sync::OnceLock::new();

impl CudaDevice {
    pub fn new() -> TensorResult<Self> {
        if let Some(d) = DEVICE.get() {
            return Ok(d.clone());
        }
        let d = Self::with_ordinal(0)?;
        Ok(DEVICE.get_or_init(|| d).clone())
    }

    pub fn with_ordinal(ordinal: i32) -> TensorResult<Self> {
        let mut ctx = std::ptr::null_mut();
        check(unsafe { ffi::tlc_init(ordinal, &mut ctx) })?;
        Ok(Self { ctx: Arc::new(CtxHandle(ctx)), ordinal })
    }

    pub(crate) fn raw(&self) -> *mut ffi::TlcCtx {
        self.ctx.0
    }

    pub fn ordinal(&self) -> i32 {
        self.ordinal
    }

    /// metal_device.rs:226
    pub fn name(&self) -> String {
        let mut buf = vec![0 as std::os::raw::c_char; 256];
        if unsafe { ffi::tlc_device_name(self.raw(), buf.as_mut_ptr(), buf.len()) } != ffi::TLC_OK {
            return String::from("CUDA device");
        }
        unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
    }

    /// metal_device.rs:195
    pub fn wait_until_completed(&self) -> TensorResult<()> {
        check(unsafe { ffi::tlc_synchronize(self.raw()) })
    }

    /// (free, total) bytes of HBM: stands in for recommended_max_working_set_size /
    /// current_allocated_size (metal_device.rs:245-256).
    pub fn mem_info(&self) -> TensorResult<(usize, usize)> {
        let (mut free, mut total) = (0usize, 0usize);
        check(unsafe { ffi::tlc_mem_info(self.raw(), &mut free, &mut total) })?;
        Ok((free, total))
    }

    /// metal_device.rs:279
    pub fn check_memory_available(&self, model_size_bytes: u64, model_name: &str) -> TensorResult<()> {
        let (free, _) = self.mem_info()?;
        if (free as u64) < model_size_bytes {
            return Err(TensorError::AllocationError(format!(
                "model '{}' needs {} bytes, {} free on {}", model_name, model_size_bytes, free, self.name())));
        }
        Ok(())
    }

    /// metal_device.rs:103: the size-class pool lives inside the library.
    pub fn buffer_pool_stats(&self) -> TensorResult<ffi::TlcPoolStats> {
        let mut s = ffi::TlcPoolStats::default();
        check(unsafe { ffi::tlc_pool_stats_get(self.raw(), &mut s) })?;
        Ok(s)
    }

    /// metal_device.rs:268
    pub fn purge_all_buffers(&self) -> TensorResult<()> {
        check(unsafe { ffi::tlc_pool_trim(self.raw(), 0) })
    }

    /// Runtime switches of the library (`tlc_set_option`), e.g. ("gemm_min_m", 32).
    pub fn set_option(&self, name: &str, value: i64) -> TensorResult<()> {
        let c = CString::new(name).map_err(|e| TensorError::InvalidOperation(e.to_string()))?;
        check(unsafe { ffi::tlc_set_option(self.raw(), c.as_ptr(), value) })
    }
}

impl PartialEq for CudaDevice {
    fn eq(&self, other: &Self) -> bool {
        self.ordinal == other.ordinal
    }
}

impl std::fmt::Debug for CudaDevice {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "CudaDevice({}: {})", self.ordinal, self.name())
    }
}
