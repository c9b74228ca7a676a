//! Quantized-resident weights.  UNCOMPILED in this repository (no Rust toolchain here).
//!
//! Upstream dequantizes every Q4_0 / Q8_0 / Q6_K tensor to f16 on ONE CPU thread while
//! loading (GGUFLoader::load, src/model/formats/gguf.rs:377-450) and uploads 2 bytes per
//! weight.  Here the GGUF blocks go to HBM as they are (regrouped into 16-row tiles on the
//! device) and `linear` runs on them directly; `dequantize()` materialises f16 on demand for
//! ops that are not on this path.

use std::ffi::CString;
use std::sync::Arc;

use half::f16;

use crate::device::cuda_buffer::CudaBuffer;
use crate::device::cuda_device::{check, CudaDevice};
use crate::device::cuda_ffi as ffi;
use crate::error::{TensorError, TensorResult};

/// GGUF type ids (src/model/formats/mmap_gguf.rs:30-45).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QType {
    F32 = 0,
    F16 = 1,
    Q4_0 = 2,
    Q8_0 = 8,
    Q6K = 14,
}

struct Handle {
    raw: *mut ffi::TlcQTensor,
    owned: bool, // false: storage belongs to a Model
}
unsafe impl Send for Handle {}
unsafe impl Sync for Handle {}
impl Drop for Handle {
    fn drop(&mut self) {
        if self.owned {
            unsafe { ffi::tlc_qtensor_destroy(self.raw) };
        }
    }
}

/// A `[rows, cols]` weight kept as GGUF blocks in HBM.  Travels through the interpreter as a
/// new `Value::QTensor(Arc<QTensor>)` variant next to `Value::TensorF16`.
#[derive(Clone)]
pub struct QTensor {
    handle: Arc<Handle>,
    device: CudaDevice,
    rows: usize,
    cols: usize,
}

impl QTensor {
    /// `blocks`: the tensor's bytes exactly as the file stores them (row-major, K fastest:
    /// dims reversed from file order, gguf.rs:288-291).
    pub fn from_blocks(device: &CudaDevice, ty: QType, rows: usize, cols: usize, blocks: &[u8]) -> TensorResult<Self> {
        let mut raw = std::ptr::null_mut();
        check(unsafe {
            ffi::tlc_qtensor_create(device.raw(), ty as i32, rows as i64, cols as i64, blocks.as_ptr() as *const _,
                                    blocks.len(), 0, 1, ffi::TLC_SPLIT_NONE, &mut raw)
        })?;
        Ok(Self { handle: Arc::new(Handle { raw, owned: true }), device: device.clone(), rows, cols })
    }

    pub(crate) fn borrowed(device: &CudaDevice, raw: *mut ffi::TlcQTensor) -> TensorResult<Self> {
        let (mut ty, mut rows, mut cols) = (0i32, 0i64, 0i64);
        check(unsafe { ffi::tlc_qtensor_info(raw, &mut ty, &mut rows, &mut cols, std::ptr::null_mut(), std::ptr::null_mut()) })?;
        Ok(Self { handle: Arc::new(Handle { raw, owned: false }), device: device.clone(), rows: rows as usize, cols: cols as usize })
    }

    pub(crate) fn raw(&self) -> *mut ffi::TlcQTensor {
        self.handle.raw
    }
    pub fn dims(&self) -> [usize; 2] {
        [self.rows, self.cols]
    }
    pub fn device(&self) -> &CudaDevice {
        &self.device
    }

    /// f16 values bit-identical to GGUFLoader::dequantize_q4_0 / _q8_0 / _q6_k
    /// (gguf.rs:22-253): for ops outside this path and for the bit-exactness tests.
    pub fn dequantize(&self) -> TensorResult<CudaBuffer<f16>> {
        let out = CudaBuffer::<f16>::new_uninit_pooled(&self.device, self.rows * self.cols)?;
        check(unsafe { ffi::tlc_dequant(self.device.raw(), self.raw(), out.as_mut_ptr()) })?;
        Ok(out)
    }
}

/// `Model<T>`'s name -> tensor map (src/model/mod.rs:39-45, :165-184) with quantized values.
pub struct CudaModel {
    raw: *mut ffi::TlcModel,
    device: CudaDevice,
}
unsafe impl Send for CudaModel {}

impl CudaModel {
    /// load_model(path) (src/interpreter/builtin_model.rs:106-131).
    pub fn load_gguf(device: &CudaDevice, path: &str) -> TensorResult<Self> {
        let c = CString::new(path).map_err(|e| TensorError::LoadError(e.to_string()))?;
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::tlc_model_load_gguf(device.raw(), c.as_ptr(), 0, 1, &mut raw) })?;
        Ok(Self { raw, device: device.clone() })
    }

    /// get_tensor(model, name) (builtin_model.rs:203-246); "Weight not found: <name>" when absent.
    pub fn get_tensor(&self, name: &str) -> TensorResult<QTensor> {
        let c = CString::new(name).map_err(|e| TensorError::LoadError(e.to_string()))?;
        let mut t = std::ptr::null_mut();
        check(unsafe { ffi::tlc_model_get(self.raw, c.as_ptr(), &mut t) })?;
        QTensor::borrowed(&self.device, t)
    }
}

impl Drop for CudaModel {
    fn drop(&mut self) {
        unsafe { ffi::tlc_model_destroy(self.raw) };
    }
}
