//! The ops of the quantized-LLM path on a CUDA device.  UNCOMPILED in this repository (no
//! Rust toolchain in the build image).
//!
//! Each function is the CUDA arm of the upstream op named in its comment: same argument
//! meaning, same defaults, same error text (the library produces the messages); results come
//! back as pooled device buffers, nothing blocks until a read-back.

use half::f16;

use crate::device::cuda_buffer::CudaBuffer;
use crate::device::cuda_device::check;
use crate::device::cuda_ffi as ffi;
use crate::error::{TensorError, TensorResult};
use crate::model::qtensor::QTensor;

/// A dense f16 tensor on the CUDA device: buffer + shape (what `Tensor<f16>` holds upstream).
pub struct CudaTensor {
    pub buf: CudaBuffer<f16>,
    pub dims: Vec<usize>,
}

impl CudaTensor {
    fn like(&self, dims: Vec<usize>) -> TensorResult<CudaTensor> {
        let n = dims.iter().product();
        Ok(CudaTensor { buf: CudaBuffer::new_uninit_pooled(self.buf.device(), n)?, dims })
    }
    fn rows_cols(&self) -> (usize, usize) {
        let cols = *self.dims.last().unwrap_or(&1);
        (self.buf.len() / cols.max(1), cols)
    }
}

/// linear(x, W[, bias]) = x . W^T (+ bias): Tensor::matmul_transposed_b, src/ops/matmul.rs:241-311,
/// builtin src/interpreter/builtin_math.rs:76-199.  W stays quantized; up to 16 rows run as the
/// fused dequant-GEMV, more rows as the tcgen05 dequant-GEMM.
pub fn linear(x: &CudaTensor, w: &QTensor, bias: Option<&CudaTensor>) -> TensorResult<CudaTensor> {
    if x.dims.len() != 2 {
        return Err(TensorError::InvalidOperation("matmul_transposed_b requires 2D tensors".to_string()));
    }
    let (m, k) = x.rows_cols();
    let y = x.like(vec![m, w.dims()[0]])?;
    check(unsafe {
        ffi::tlc_linear(x.buf.device().raw(), w.raw(), x.buf.as_ptr(), m as i32, k as i64, y.buf.as_mut_ptr(),
                        bias.map_or(std::ptr::null(), |b| b.buf.as_ptr()))
    })?;
    Ok(y)
}

/// matmul(a, b): Tensor::matmul, src/ops/matmul.rs:13-75.
pub fn matmul(a: &CudaTensor, b: &CudaTensor) -> TensorResult<CudaTensor> {
    if a.dims.len() != 2 || b.dims.len() != 2 {
        return Err(TensorError::InvalidOperation("matmul requires 2D tensors".to_string()));
    }
    let y = a.like(vec![a.dims[0], b.dims[1]])?;
    check(unsafe {
        ffi::tlc_matmul(a.buf.device().raw(), a.buf.as_ptr(), b.buf.as_ptr(), y.buf.as_mut_ptr(), a.dims[0] as i32,
                        a.dims[1] as i32, b.dims[0] as i32, b.dims[1] as i32)
    })?;
    Ok(y)
}

/// rms_norm(x, weight[, eps = 1e-6]): Tensor::rms_norm, src/ops/normalization.rs:42-88.
pub fn rms_norm(x: &CudaTensor, weight: &CudaTensor, eps: f32) -> TensorResult<CudaTensor> {
    let (rows, d) = x.rows_cols();
    let y = x.like(x.dims.clone())?;
    check(unsafe {
        ffi::tlc_rms_norm(x.buf.device().raw(), x.buf.as_ptr(), weight.buf.as_ptr(), y.buf.as_mut_ptr(), rows as i32,
                          d as i32, eps)
    })?;
    Ok(y)
}

/// rope(x[, position_offset]): Tensor::rope, src/ops/rope.rs:71-118; x is [..., seq, heads, head_dim].
pub fn rope(x: &CudaTensor, position_offset: usize) -> TensorResult<CudaTensor> {
    if x.dims.len() < 3 {
        return Err(TensorError::InvalidOperation("RoPE requires at least 3D tensor [seq, heads, head_dim]".to_string()));
    }
    let (heads, d) = (x.dims[x.dims.len() - 2], x.dims[x.dims.len() - 1]);
    let seq = x.buf.len() / (heads * d);
    let y = x.like(x.dims.clone())?;
    check(unsafe {
        ffi::tlc_rope(x.buf.device().raw(), x.buf.as_ptr(), y.buf.as_mut_ptr(), seq as i32, heads as i32, d as i32,
                      position_offset as i32, 10000, std::ptr::null())
    })?;
    Ok(y)
}

/// rope(x, cos, sin): Tensor::rope_candle, src/ops/rope.rs:18-65.  cos / sin are
/// [max_seq_len, cols]; cols = head_dim is the upstream table, cols = head_dim / 2 one column
/// per pair (see tlc_rope_table in tlcuda.h for what each means).
pub fn rope_candle(x: &CudaTensor, cos: &CudaTensor, sin: &CudaTensor) -> TensorResult<CudaTensor> {
    if x.dims.len() != 3 {
        return Err(TensorError::InvalidOperation(format!(
            "rope_candle requires 3D tensor [seq_len, n_heads, head_dim], got {}D", x.dims.len())));
    }
    if cos.dims.len() != 2 || sin.dims.len() != 2 || cos.dims != sin.dims {
        return Err(TensorError::InvalidOperation(format!(
            "cos/sin must be 2D [max_seq_len, head_dim], got cos: {}D, sin: {}D", cos.dims.len(), sin.dims.len())));
    }
    let y = x.like(x.dims.clone())?;
    check(unsafe {
        ffi::tlc_rope_table(x.buf.device().raw(), x.buf.as_ptr(), cos.buf.as_ptr(), sin.buf.as_ptr(), y.buf.as_mut_ptr(),
                            x.dims[0] as i32, x.dims[1] as i32, x.dims[2] as i32, cos.dims[0] as i32, cos.dims[1] as i32)
    })?;
    Ok(y)
}

macro_rules! unary {
    ($name:ident, $ffi:ident, $doc:literal) => {
        #[doc = $doc]
        pub fn $name(x: &CudaTensor) -> TensorResult<CudaTensor> {
            let y = x.like(x.dims.clone())?;
            check(unsafe { ffi::$ffi(x.buf.device().raw(), x.buf.as_ptr(), y.buf.as_mut_ptr(), x.buf.len()) })?;
            Ok(y)
        }
    };
}
macro_rules! binary {
    ($name:ident, $ffi:ident, $doc:literal) => {
        #[doc = $doc]
        pub fn $name(a: &CudaTensor, b: &CudaTensor) -> TensorResult<CudaTensor> {
            if a.dims != b.dims {
                return Err(TensorError::InvalidOperation(format!("shape mismatch: {:?} vs {:?}", a.dims, b.dims)));
            }
            let y = a.like(a.dims.clone())?;
            check(unsafe {
                ffi::$ffi(a.buf.device().raw(), a.buf.as_ptr(), b.buf.as_ptr(), y.buf.as_mut_ptr(), a.buf.len())
            })?;
            Ok(y)
        }
    };
}
unary!(sigmoid, tlc_sigmoid, "Tensor::sigmoid, src/ops/activations.rs:239-266.");
binary!(mul, tlc_mul, "Tensor::mul, src/ops/elementwise.rs:232-330.");
binary!(add, tlc_add, "Tensor::add, src/ops/elementwise.rs:48-140.");

/// softmax(x) over the last dim: Tensor::softmax, src/ops/activations.rs:107-229 (the builtin
/// ignores its `dim` argument, src/interpreter/builtin_sampling.rs:39-45).
pub fn softmax(x: &CudaTensor) -> TensorResult<CudaTensor> {
    let (rows, last) = x.rows_cols();
    let y = x.like(x.dims.clone())?;
    check(unsafe { ffi::tlc_softmax(x.buf.device().raw(), x.buf.as_ptr(), y.buf.as_mut_ptr(), rows as i32, last as i32) })?;
    Ok(y)
}

/// embedding(table, ids): src/interpreter/builtin_nn.rs:627-811; ids are checked on the host
/// ("Index out of bounds: index i, size n", :681-688).
pub fn embedding(table: &CudaTensor, ids: &[i32]) -> TensorResult<CudaTensor> {
    let (vocab, d) = (table.dims[0], table.dims[1]);
    let y = table.like(vec![ids.len(), d])?;
    check(unsafe {
        ffi::tlc_embedding(table.buf.device().raw(), table.buf.as_ptr(), vocab as i32, d as i32, ids.as_ptr(),
                           ids.len() as i32, y.buf.as_mut_ptr())
    })?;
    Ok(y)
}
