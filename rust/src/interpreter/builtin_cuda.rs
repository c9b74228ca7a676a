//! Builtin arms that pick the CUDA path.  UNCOMPILED in this repository (no Rust toolchain in
//! the build image); written as the patch a maintainer applies to the interpreter.
//!
//! Upstream dispatches `linear`, `rms_norm`, `rope`, ... by the `Value` variant of the
//! operands (src/interpreter/builtin_math.rs:76-199, builtin_nn.rs:44-151,
//! builtin_tensor.rs:514-567): both operands must be the same variant.  Two new variants join
//! `Value::TensorF16` / `Value::TensorF32`:
//!
//!     Value::CudaTensor(Arc<CudaTensor>)   // dense f16 on the CUDA device
//!     Value::QTensor(Arc<QTensor>)         // GGUF blocks resident in HBM (get_tensor on a CUDA model)
//!
//! and each builtin gets one more match arm in front of the existing ones.

use std::sync::Arc;

use crate::interpreter::value::Value;
use crate::interpreter::{Interpreter, RuntimeError, RuntimeResult};
use crate::ops::cuda_ops as ops;
use crate::ast::TensorExpr;

impl Interpreter {
    /// linear(x, weight[, bias]) -- the arm added to eval_linear (builtin_math.rs:76-199).
    /// Returns Ok(None) when the operands are not on the CUDA path, so that the caller falls
    /// through to the upstream arms.
    pub(crate) fn eval_linear_cuda(&mut self, args: &[TensorExpr]) -> RuntimeResult<Option<Value>> {
        if args.len() < 2 || args.len() > 3 {
            return Err(RuntimeError::TypeError(format!(
                "linear() expects 2-3 arguments (x, weight, [bias]), got {}", args.len())));
        }
        let _start = std::time::Instant::now();
        let x = self.eval_expr(&args[0])?;
        let w = self.eval_expr(&args[1])?;
        let (x, w) = match (x, w) {
            (Value::CudaTensor(x), Value::QTensor(w)) => (x, w),
            _ => return Ok(None),
        };
        let bias = if args.len() == 3 {
            match self.eval_expr(&args[2])? {
                Value::CudaTensor(b) => Some(b),
                _ => return Err(RuntimeError::TypeError("linear() bias must be a tensor on the same device".to_string())),
            }
        } else {
            None
        };
        let y = ops::linear(&x, &w, bias.as_deref()).map_err(RuntimeError::TensorError)?;
        if std::env::var("TL_PERF").is_ok() {
            // upstream prints host wall time per op (builtin_math.rs:190-197); the device-side
            // per-phase times of a whole decode step come from tlc_llama_step_trace
            eprintln!("[PERF] linear(q, cuda): {:.3}ms", _start.elapsed().as_secs_f64() * 1000.0);
        }
        Ok(Some(Value::CudaTensor(Arc::new(y))))
    }

    /// rms_norm(x, weight[, eps]) -- the arm added to eval_rms_norm (builtin_nn.rs:44-151);
    /// eps defaults to 1e-6 (:83-92).
    pub(crate) fn eval_rms_norm_cuda(&mut self, args: &[TensorExpr]) -> RuntimeResult<Option<Value>> {
        if args.len() < 2 || args.len() > 3 {
            return Err(RuntimeError::TypeError(format!(
                "rms_norm() expects 2-3 arguments (tensor, weight, [eps]), got {}", args.len())));
        }
        let (x, w) = match (self.eval_expr(&args[0])?, self.eval_expr(&args[1])?) {
            (Value::CudaTensor(x), Value::CudaTensor(w)) => (x, w),
            _ => return Ok(None),
        };
        let eps = if args.len() == 3 {
            match self.eval_expr(&args[2])? {
                Value::Float(f) => f as f32,
                Value::Integer(i) => i as f32,
                _ => return Err(RuntimeError::TypeError("rms_norm() eps must be a number".to_string())),
            }
        } else {
            1e-6
        };
        let y = ops::rms_norm(&x, &w, eps).map_err(RuntimeError::TensorError)?;
        Ok(Some(Value::CudaTensor(Arc::new(y))))
    }

    /// rope(x[, position_offset]) and rope(x, cos, sin) -- the arms added to eval_rope
    /// (builtin_tensor.rs:514-567, :634-722).
    pub(crate) fn eval_rope_cuda(&mut self, args: &[TensorExpr]) -> RuntimeResult<Option<Value>> {
        if args.is_empty() || args.len() > 3 {
            return Err(RuntimeError::TypeError(format!(
                "rope() expects 1-3 arguments (tensor, [position_offset] OR tensor, cos, sin), got {}", args.len())));
        }
        let x = match self.eval_expr(&args[0])? {
            Value::CudaTensor(x) => x,
            _ => return Ok(None),
        };
        let y = if args.len() == 3 {
            match (self.eval_expr(&args[1])?, self.eval_expr(&args[2])?) {
                (Value::CudaTensor(c), Value::CudaTensor(s)) => ops::rope_candle(&x, &c, &s),
                _ => return Err(RuntimeError::TypeError("rope() cos/sin must be tensors on the same device".to_string())),
            }
        } else {
            let offset = if args.len() == 2 {
                match self.eval_expr(&args[1])? {
                    Value::Float(f) => f as usize,
                    Value::Integer(i) => i as usize,
                    _ => return Err(RuntimeError::TypeError("rope() position_offset must be a scalar integer".to_string())),
                }
            } else {
                0
            };
            ops::rope(&x, offset)
        }
        .map_err(RuntimeError::TensorError)?;
        Ok(Some(Value::CudaTensor(Arc::new(y))))
    }
}
