//! Device buffer: the counterpart of `MetalBuffer<T>` (src/device/metal_buffer.rs).
//! UNCOMPILED in this repository (no Rust toolchain in the build image).
//!
//! Ownership follows upstream: the buffer is shared as `Arc`, and the LAST owner hands the
//! allocation back to the library's size-class pool on drop (metal_buffer.rs:246-291,
//! buffer_pool.rs:426-499).  The pool never zeroes reused memory (buffer_pool.rs:222-230).

use std::marker::PhantomData;
use std::os::raw::c_void;
use std::sync::Arc;

use crate::device::cuda_device::{check, CudaDevice};
use crate::device::cuda_ffi as ffi;
use crate::error::TensorResult;
use crate::tensor::FloatType;

struct Allocation {
    buf: *mut ffi::TlcBuf,
}
unsafe impl Send for Allocation {}
unsafe impl Sync for Allocation {}
impl Drop for Allocation {
    fn drop(&mut self) {
        unsafe { ffi::tlc_free(self.buf) }; // back to its size class
    }
}

#[derive(Clone)]
pub struct CudaBuffer<T: FloatType> {
    alloc: Arc<Allocation>,
    device: CudaDevice,
    length: usize,
    _marker: PhantomData<T>,
}

impl<T: FloatType> CudaBuffer<T> {
    /// metal_buffer.rs:213 (`new_uninit_pooled`): contents are whatever the last user left.
    pub fn new_uninit_pooled(device: &CudaDevice, length: usize) -> TensorResult<Self> {
        let mut buf = std::ptr::null_mut();
        check(unsafe { ffi::tlc_alloc(device.raw(), length.max(1) * std::mem::size_of::<T>(), &mut buf) })?;
        Ok(Self { alloc: Arc::new(Allocation { buf }), device: device.clone(), length, _marker: PhantomData })
    }

    /// metal_buffer.rs:37 / :226 (`from_slice`, `from_vec_pooled`): host to device.
    pub fn from_slice(device: &CudaDevice, data: &[T]) -> TensorResult<Self> {
        let b = Self::new_uninit_pooled(device, data.len())?;
        check(unsafe {
            ffi::tlc_upload(device.raw(), b.as_mut_ptr(), data.as_ptr() as *const c_void, std::mem::size_of_val(data))
        })?;
        Ok(b)
    }

    pub fn from_vec_pooled(device: &CudaDevice, data: &[T]) -> TensorResult<Self> {
        Self::from_slice(device, data)
    }

    /// metal_buffer.rs:113 (`to_vec`): waits for the stream, then device to host.  The one
    /// blocking point of the op path upstream (`sync_and_read*`, tensor_io.rs:111-114).
    pub fn to_vec(&self) -> TensorResult<Vec<T>> {
        let mut out = Vec::<T>::with_capacity(self.length);
        check(unsafe {
            ffi::tlc_download(self.device.raw(), out.as_mut_ptr() as *mut c_void, self.as_ptr(),
                              self.length * std::mem::size_of::<T>())
        })?;
        unsafe { out.set_len(self.length) };
        Ok(out)
    }

    pub fn len(&self) -> usize {
        self.length
    }
    pub fn is_empty(&self) -> bool {
        self.length == 0
    }
    pub fn byte_length(&self) -> usize {
        self.length * std::mem::size_of::<T>()
    }
    pub fn device(&self) -> &CudaDevice {
        &self.device
    }
    pub fn as_ptr(&self) -> *const c_void {
        unsafe { ffi::tlc_buf_ptr(self.alloc.buf) as *const c_void }
    }
    pub fn as_mut_ptr(&self) -> *mut c_void {
        unsafe { ffi::tlc_buf_ptr(self.alloc.buf) }
    }
}
