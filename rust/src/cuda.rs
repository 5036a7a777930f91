//! `--backend cuda`: the B200 (sm_100a) backend for the Heron forward path, beside `src/metal.rs`.
//!
//! A safe wrapper over `ullis-cuda-sys` (the raw FFI of `libullis_cuda.so`).  `CudaRuntime` carries
//! the methods of `MetalRuntime` that the forward path, the streamed cross-entropy and the optimiser
//! steps use - same names, same argument meaning, same `bail!` wording for shape errors - so the
//! `*_on` methods of `src/model.rs` can take a CUDA arm next to their Metal arm.  `CudaHeron` is the
//! addition that suits a discrete GPU: the whole model lives on the device, token ids go in and a
//! loss (or logits) comes out, with no host round trip per operator.
//!
//! There is no CPU fallback in here: without a CUDA device `CudaRuntime::new` is an error, as
//! `--backend metal` is on a machine without Metal (`src/main.rs:675-678`).
//!
//! This file is written against `include/ullis_cuda.h` and has NOT been compiled: the machine the
//! CUDA backend is developed on has no rustc.  Every entry point it calls is exercised through the
//! same C ABI by the Python mirror (`ullis_b200/cuda.py`) and its GPU tests, and a CPU test checks
//! that every `sys::` name used here is declared by the header with the same number of arguments.

// The crate denies `unsafe_code`; like `src/metal/ffi.rs` for Metal, this module is the one audited
// place of the CUDA backend where calls cross the FFI.  Every `unsafe` block below is a single call
// into `ullis-cuda-sys` whose pointer arguments were length-checked just above it.
#![allow(unsafe_code)]

use core::ffi::CStr;
use core::ptr;

use anyhow::{Result, anyhow, bail};
use ullis_cuda_sys as sys;

use crate::precision::Fp16;

/// `ignore_id` that supervises every in-range target (`CE_NO_IGNORE`, `src/model.rs:24`).
pub const CE_NO_IGNORE: u32 = u32::MAX;

/// Arithmetic of the linears and LayerNorm (`ULLIS_CUDA_MODE_*`).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum CudaMode {
    /// tcgen05 tensor-core GEMMs, warp-shuffle LayerNorm: within 1e-2 relative of the CPU backend.
    Fast,
    /// The CPU backend's summation order on CUDA cores: bit-identical activations and logits.
    Exact,
}

/// Checked dimensions of one packed or FP16 projection (`LinearDispatchShape`, `src/metal.rs:62-88`).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub struct LinearDispatchShape {
    pub rows: usize,
    pub in_features: usize,
    pub out_features: usize,
}

impl LinearDispatchShape {
    pub fn new(rows: usize, in_features: usize, out_features: usize) -> Result<Self> {
        if rows == 0 || out_features == 0 || in_features == 0 {
            bail!("CUDA linear dispatch dimensions must be non-zero");
        }
        if rows.checked_mul(out_features).is_none() || in_features.checked_mul(out_features).is_none() {
            bail!("CUDA linear shape overflow");
        }
        Ok(Self { rows, in_features, out_features })
    }

    pub fn packed_words(self) -> usize {
        (self.in_features * self.out_features).div_ceil(32)
    }
}

/// `RosaQkvForward` (`src/metal.rs:253-256`).
#[derive(Clone, Debug, PartialEq)]
pub struct RosaQkvForward {
    pub idx: Vec<u8>,
    pub out: Vec<f32>,
}

/// `RosaQkvBlockForward` (`src/metal.rs:260-269`) without the Metal-resident tapes.
#[derive(Clone, Debug, PartialEq)]
pub struct RosaQkvBlockForward {
    pub idx: Vec<u8>,
    pub y: Vec<f32>,
    pub out: Vec<f32>,
}

/// `LayerNormBackward` (`src/metal.rs:229-233`).
#[derive(Clone, Debug, PartialEq)]
pub struct LayerNormBackward {
    pub input_gradient: Vec<f32>,
    pub weight_gradient: Vec<f32>,
    pub bias_gradient: Vec<f32>,
}

/// Forward part of `StreamedCrossEntropy` (`src/metal.rs:325-331`).
#[derive(Clone, Debug, PartialEq)]
pub struct StreamedCrossEntropy {
    pub mean_loss: f32,
    pub n_valid: u64,
    pub row_loss: Vec<f32>,
}

/// One packed linear as the C ABI takes it: sign words in checkpoint order, FP16 bits of the row
/// scales and of the optional bias (`PackedBinaryLinear`, `src/model.rs:560-567`, `672-682`).
#[derive(Clone, Copy, Debug)]
pub struct PackedLinearRef<'a> {
    pub bits: &'a [u32],
    pub scale: &'a [u16],
    pub bias: Option<&'a [u16]>,
}

fn fp16_bits(values: &[f32]) -> Vec<u16> {
    values.iter().map(|&v| Fp16::from_f32(v).to_bits()).collect()
}

fn last_error(rt: *const sys::ullis_cuda_runtime) -> String {
    // SAFETY: the library returns a NUL-terminated string that stays valid until the next call on `rt`.
    unsafe { CStr::from_ptr(sys::ullis_cuda_last_error(rt)) }
        .to_string_lossy()
        .into_owned()
}

fn opt_ptr(bias: Option<&[u16]>) -> *const u16 {
    bias.map_or(ptr::null(), <[u16]>::as_ptr)
}

/// One CUDA device, one stream.  `!Send + !Sync` through the raw pointer, like `MetalRuntime`
/// with its `RefCell` scratch pool (`src/metal.rs:452-457`): use it from the thread that made it.
#[derive(Debug)]
pub struct CudaRuntime {
    raw: *mut sys::ullis_cuda_runtime,
}

impl CudaRuntime {
    /// `MetalRuntime::new` (`src/metal.rs:466`).  Fails when the machine has no usable CUDA device.
    pub fn new(device: i32) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer; the library writes a handle or leaves it null.
        let rc = unsafe { sys::ullis_cuda_runtime_create(device, &mut raw) };
        if rc != sys::ULLIS_CUDA_OK || raw.is_null() {
            bail!("{}", last_error(ptr::null()));
        }
        Ok(Self { raw })
    }

    fn check(&self, rc: i32) -> Result<()> {
        if rc == sys::ULLIS_CUDA_OK {
            Ok(())
        } else {
            Err(anyhow!("{}", last_error(self.raw)))
        }
    }

    pub fn set_mode(&self, mode: CudaMode) -> Result<()> {
        let m = match mode {
            CudaMode::Fast => sys::ULLIS_CUDA_MODE_FAST,
            CudaMode::Exact => sys::ULLIS_CUDA_MODE_EXACT,
        };
        // SAFETY: `self.raw` is a live runtime handle for the whole life of `self`.
        self.check(unsafe { sys::ullis_cuda_runtime_set_mode(self.raw, m) })
    }

    /// `MetalRuntime::synchronize` (`src/metal.rs:598`).
    pub fn synchronize(&self) -> Result<()> {
        // SAFETY: live handle.
        self.check(unsafe { sys::ullis_cuda_runtime_synchronize(self.raw) })
    }

    /// Whether the device is an sm_100 part (the tensor-core kernels need one).
    pub fn is_sm100(&self) -> bool {
        // SAFETY: live handle.
        unsafe { sys::ullis_cuda_runtime_is_sm100(self.raw) == 1 }
    }

    /// Kernels launched through this runtime so far.
    pub fn launch_count(&self) -> u64 {
        // SAFETY: live handle.
        unsafe { sys::ullis_cuda_runtime_launch_count(self.raw) }
    }

    /// Records a CUDA event behind every launch from now on (or stops doing so).
    pub fn kernel_timing(&self, enabled: bool) -> Result<()> {
        // SAFETY: live handle.
        self.check(unsafe { sys::ullis_cuda_runtime_kernel_timing(self.raw, i32::from(enabled)) })
    }

    /// `(kernel name, total milliseconds, launches)` since timing was switched on.
    pub fn kernel_times(&self) -> Result<Vec<(String, f32, u32)>> {
        let mut needed = 0_usize;
        // SAFETY: a null buffer of length 0 only asks for the size.
        self.check(unsafe { sys::ullis_cuda_runtime_kernel_names(self.raw, ptr::null_mut(), 0, &mut needed) })?;
        let mut buf = vec![0_u8; needed.max(1)];
        // SAFETY: `buf` holds `buf.len()` writable bytes.
        self.check(unsafe {
            sys::ullis_cuda_runtime_kernel_names(self.raw, buf.as_mut_ptr().cast(), buf.len(), &mut needed)
        })?;
        let text = String::from_utf8_lossy(&buf[..buf.iter().position(|&b| b == 0).unwrap_or(buf.len())]).into_owned();
        let mut out = Vec::new();
        for name in text.lines().filter(|l| !l.is_empty()) {
            let c_name = std::ffi::CString::new(name)?;
            let (mut ms, mut launches) = (0.0_f32, 0_u32);
            // SAFETY: `c_name` is NUL-terminated; the two out-pointers are valid.
            self.check(unsafe {
                sys::ullis_cuda_runtime_kernel_time(self.raw, c_name.as_ptr(), &mut ms, &mut launches)
            })?;
            out.push((name.to_owned(), ms, launches));
        }
        Ok(out)
    }

    /// `MetalRuntime::residual_add` (`src/metal.rs:1078`).
    pub fn residual_add(&self, residual: &[f32], update: &[f32]) -> Result<Vec<f32>> {
        if residual.len() != update.len() {
            bail!("residual add length mismatch");
        }
        let mut out = vec![0.0_f32; residual.len()];
        if residual.is_empty() {
            return Ok(out);
        }
        // SAFETY: three buffers of `residual.len()` floats.
        self.check(unsafe {
            sys::ullis_cuda_residual_add(self.raw, residual.as_ptr(), update.as_ptr(), out.as_mut_ptr(), residual.len())
        })?;
        Ok(out)
    }

    /// `MetalRuntime::time_shift_delta` (`src/metal.rs:1103`); `src/model.rs:186-212`.
    pub fn time_shift_delta(&self, input: &[f32], rows: usize, time: usize, channels: usize) -> Result<Vec<f32>> {
        if rows.checked_mul(channels) != Some(input.len()) || time == 0 || rows % time != 0 {
            bail!("time-shift input shape mismatch");
        }
        let mut out = vec![0.0_f32; input.len()];
        // SAFETY: `input` and `out` hold rows * channels floats.
        self.check(unsafe {
            sys::ullis_cuda_time_shift_delta(self.raw, input.as_ptr(), out.as_mut_ptr(), rows, time, channels)
        })?;
        Ok(out)
    }

    /// `MetalRuntime::sign_pack_bits` (`src/metal.rs:1142`): bit = x > 0, 32 per word, LSB first.
    pub fn sign_pack_bits(&self, input: &[f32]) -> Result<Vec<u32>> {
        if input.is_empty() {
            return Ok(Vec::new());
        }
        let mut bits = vec![0_u32; input.len().div_ceil(32)];
        // SAFETY: `bits` holds ceil(n / 32) words.
        self.check(unsafe { sys::ullis_cuda_sign_pack_bits(self.raw, input.as_ptr(), bits.as_mut_ptr(), input.len()) })?;
        Ok(bits)
    }

    /// `MetalRuntime::rosa_qkv_1bit_fwd` (`src/metal.rs:1168`): packed `[B, T, C]` bit planes in,
    /// idx bit-exact with `rosa_qkv_batch` and `out = (2 idx - 1) e` out.  `e` is widened FP16.
    pub fn rosa_qkv_1bit_fwd(
        &self,
        q_bits: &[u32],
        k_bits: &[u32],
        v_bits: &[u32],
        e: &[f32],
        batch: usize,
        time: usize,
        channels: usize,
    ) -> Result<RosaQkvForward> {
        let n = batch
            .checked_mul(time)
            .and_then(|bt| bt.checked_mul(channels))
            .ok_or_else(|| anyhow!("ROSA dispatch shape overflow"))?;
        if n == 0 {
            bail!("ROSA dispatch dimensions must be non-zero");
        }
        let words = n.div_ceil(32);
        if q_bits.len() != words || k_bits.len() != words || v_bits.len() != words || e.len() != channels {
            bail!("ROSA QKV input shape mismatch");
        }
        let e_bits = fp16_bits(e);
        let mut idx = vec![0_u8; n];
        let mut out = vec![0.0_f32; n];
        // SAFETY: plane, e, idx and out lengths were checked against batch * time * channels above.
        self.check(unsafe {
            sys::ullis_cuda_rosa_qkv_1bit_fwd(
                self.raw,
                q_bits.as_ptr(),
                k_bits.as_ptr(),
                v_bits.as_ptr(),
                e_bits.as_ptr(),
                idx.as_mut_ptr(),
                out.as_mut_ptr(),
                batch,
                time,
                channels,
            )
        })?;
        Ok(RosaQkvForward { idx, out })
    }

    /// `MetalRuntime::rosa_qkv_1bit_bwd_e` (`src/metal.rs:1258`); `rosa_e_grad` (`src/model.rs:1608-1634`).
    pub fn rosa_qkv_1bit_bwd_e(
        &self,
        output_gradient: &[f32],
        idx: &[u8],
        batch: usize,
        time: usize,
        channels: usize,
    ) -> Result<Vec<f32>> {
        let n = batch * time * channels;
        if output_gradient.len() != n || idx.len() != n {
            bail!("ROSA e-gradient shape mismatch");
        }
        let mut g_e = vec![0.0_f32; channels];
        // SAFETY: lengths checked above; g_e holds `channels` floats.
        self.check(unsafe {
            sys::ullis_cuda_rosa_qkv_1bit_bwd_e(
                self.raw,
                output_gradient.as_ptr(),
                idx.as_ptr(),
                batch,
                time,
                channels,
                g_e.as_mut_ptr(),
            )
        })?;
        Ok(g_e)
    }

    /// `MetalRuntime::rosa_block_forward` (`src/metal.rs:1334`); `RwkvRosaQkv1Bit::forward`
    /// (`src/model.rs:1284-1318`): time-shift mixes, Q/K/V, sign bits, automaton, `(2 idx - 1) e`, O.
    #[allow(clippy::too_many_arguments)]
    pub fn rosa_block_forward(
        &self,
        x: &[f32],
        mix_q: &[u16],
        mix_k: &[u16],
        mix_v: &[u16],
        q: PackedLinearRef<'_>,
        k: PackedLinearRef<'_>,
        v: PackedLinearRef<'_>,
        e: &[u16],
        o: PackedLinearRef<'_>,
        batch: usize,
        time: usize,
        channels: usize,
    ) -> Result<RosaQkvBlockForward> {
        let n = batch * time * channels;
        let words = (channels * channels).div_ceil(32);
        let vec_ok = |s: &[u16]| s.len() == channels;
        let lin_ok = |l: &PackedLinearRef<'_>| {
            l.bits.len() == words && vec_ok(l.scale) && l.bias.is_some_and(|b| b.len() == channels)
        };
        if x.len() != n || !vec_ok(mix_q) || !vec_ok(mix_k) || !vec_ok(mix_v) || !vec_ok(e) {
            bail!("ROSA block input shape mismatch");
        }
        if !(lin_ok(&q) && lin_ok(&k) && lin_ok(&v) && lin_ok(&o)) {
            bail!("ROSA block packed-linear shape mismatch");
        }
        let mut idx = vec![0_u8; n];
        let mut y = vec![0.0_f32; n];
        let mut out = vec![0.0_f32; n];
        // SAFETY: every slice length was checked against the dimensions passed along.
        self.check(unsafe {
            sys::ullis_cuda_rosa_block_forward(
                self.raw,
                x.as_ptr(),
                mix_q.as_ptr(),
                mix_k.as_ptr(),
                mix_v.as_ptr(),
                q.bits.as_ptr(),
                q.scale.as_ptr(),
                opt_ptr(q.bias),
                k.bits.as_ptr(),
                k.scale.as_ptr(),
                opt_ptr(k.bias),
                v.bits.as_ptr(),
                v.scale.as_ptr(),
                opt_ptr(v.bias),
                e.as_ptr(),
                o.bits.as_ptr(),
                o.scale.as_ptr(),
                opt_ptr(o.bias),
                batch,
                time,
                channels,
                ptr::null_mut(),
                ptr::null_mut(),
                ptr::null_mut(),
                idx.as_mut_ptr(),
                y.as_mut_ptr(),
                out.as_mut_ptr(),
            )
        })?;
        Ok(RosaQkvBlockForward { idx, y, out })
    }

    /// `MetalRuntime::cmix_relu2` (`src/metal.rs:1542`).
    pub fn cmix_relu2(&self, input: &[f32]) -> Result<Vec<f32>> {
        let mut out = vec![0.0_f32; input.len()];
        if input.is_empty() {
            return Ok(out);
        }
        // SAFETY: both buffers hold `input.len()` floats.
        self.check(unsafe { sys::ullis_cuda_cmix_relu2(self.raw, input.as_ptr(), out.as_mut_ptr(), input.len()) })?;
        Ok(out)
    }

    /// `MetalRuntime::cmix_relu2_backward` (`src/metal.rs:1546`).
    pub fn cmix_relu2_backward(&self, input: &[f32], output_gradient: &[f32]) -> Result<Vec<f32>> {
        if input.len() != output_gradient.len() {
            bail!("relu2 backward length mismatch");
        }
        let mut gx = vec![0.0_f32; input.len()];
        if input.is_empty() {
            return Ok(gx);
        }
        // SAFETY: three buffers of `input.len()` floats.
        self.check(unsafe {
            sys::ullis_cuda_cmix_relu2_backward(
                self.raw,
                input.as_ptr(),
                output_gradient.as_ptr(),
                gx.as_mut_ptr(),
                input.len(),
            )
        })?;
        Ok(gx)
    }

    /// `MetalRuntime::layer_norm` (`src/metal.rs:1590`); `LayerNorm::forward` (`src/model.rs:259-276`).
    /// `weight` / `bias` are the widened FP16 parameters, as the Metal method takes them.
    pub fn layer_norm(&self, input: &[f32], weight: &[f32], bias: &[f32], rows: usize, channels: usize) -> Result<Vec<f32>> {
        if rows.checked_mul(channels) != Some(input.len()) || weight.len() != channels || bias.len() != channels {
            bail!("LayerNorm input shape mismatch");
        }
        let (w, b) = (fp16_bits(weight), fp16_bits(bias));
        let mut out = vec![0.0_f32; input.len()];
        // SAFETY: lengths checked above.
        self.check(unsafe {
            sys::ullis_cuda_layer_norm(self.raw, input.as_ptr(), w.as_ptr(), b.as_ptr(), out.as_mut_ptr(), rows, channels)
        })?;
        Ok(out)
    }

    /// `MetalRuntime::layer_norm_backward` (`src/metal.rs:1628`).
    pub fn layer_norm_backward(
        &self,
        input: &[f32],
        output_gradient: &[f32],
        weight: &[f32],
        rows: usize,
        channels: usize,
    ) -> Result<LayerNormBackward> {
        if rows.checked_mul(channels) != Some(input.len()) || output_gradient.len() != input.len() || weight.len() != channels {
            bail!("LayerNorm backward shape mismatch");
        }
        let w = fp16_bits(weight);
        let mut gx = vec![0.0_f32; input.len()];
        let mut gw = vec![0.0_f32; channels];
        let mut gb = vec![0.0_f32; channels];
        // SAFETY: lengths checked above.
        self.check(unsafe {
            sys::ullis_cuda_layer_norm_backward(
                self.raw,
                input.as_ptr(),
                output_gradient.as_ptr(),
                w.as_ptr(),
                rows,
                channels,
                gx.as_mut_ptr(),
                gw.as_mut_ptr(),
                gb.as_mut_ptr(),
            )
        })?;
        Ok(LayerNormBackward { input_gradient: gx, weight_gradient: gw, bias_gradient: gb })
    }

    /// `MetalRuntime::binary_linear` (`src/metal.rs:1705`); `PackedBinaryLinear::forward`
    /// (`src/model.rs:724-742`).  `scale` / `bias` are the widened FP16 parameters.
    pub fn binary_linear(
        &self,
        input: &[f32],
        bits: &[u32],
        scale: &[f32],
        bias: Option<&[f32]>,
        shape: LinearDispatchShape,
    ) -> Result<Vec<f32>> {
        if shape.rows.checked_mul(shape.in_features) != Some(input.len())
            || bits.len() != shape.packed_words()
            || scale.len() != shape.out_features
            || bias.is_some_and(|b| b.len() != shape.out_features)
        {
            bail!("packed linear input shape mismatch");
        }
        let scale_bits = fp16_bits(scale);
        let bias_bits = bias.map(fp16_bits);
        let mut out = vec![0.0_f32; shape.rows * shape.out_features];
        // SAFETY: lengths checked above; a missing bias crosses as a null pointer.
        self.check(unsafe {
            sys::ullis_cuda_binary_linear(
                self.raw,
                input.as_ptr(),
                bits.as_ptr(),
                scale_bits.as_ptr(),
                opt_ptr(bias_bits.as_deref()),
                out.as_mut_ptr(),
                shape.rows,
                shape.in_features,
                shape.out_features,
            )
        })?;
        Ok(out)
    }

    /// `MetalRuntime::cmix_block_forward` (`src/metal.rs:1891`); `RwkvCMixX070::forward`
    /// (`src/model.rs:987-1001`).  Returns the block output (the Metal method's `out`).
    #[allow(clippy::too_many_arguments)]
    pub fn cmix_block_forward(
        &self,
        x: &[f32],
        mix: &[u16],
        key_bits: &[u32],
        key_scale: &[u16],
        value_weight: &[u16],
        batch: usize,
        time: usize,
        d_model: usize,
        dim_ffn: usize,
    ) -> Result<Vec<f32>> {
        if x.len() != batch * time * d_model
            || mix.len() != d_model
            || key_bits.len() != (d_model * dim_ffn).div_ceil(32)
            || key_scale.len() != dim_ffn
            || value_weight.len() != d_model * dim_ffn
        {
            bail!("CMix block input shape mismatch");
        }
        let mut out = vec![0.0_f32; x.len()];
        // SAFETY: lengths checked above.
        self.check(unsafe {
            sys::ullis_cuda_cmix_block_forward(
                self.raw,
                x.as_ptr(),
                mix.as_ptr(),
                key_bits.as_ptr(),
                key_scale.as_ptr(),
                value_weight.as_ptr(),
                batch,
                time,
                d_model,
                dim_ffn,
                out.as_mut_ptr(),
            )
        })?;
        Ok(out)
    }

    /// `MetalRuntime::fp16_linear` (`src/metal.rs:2790`); `Fp16Linear::forward` (`src/model.rs:419-436`).
    pub fn fp16_linear(&self, input: &[f32], weight: &[f32], shape: LinearDispatchShape) -> Result<Vec<f32>> {
        if shape.rows.checked_mul(shape.in_features) != Some(input.len())
            || weight.len() != shape.in_features * shape.out_features
        {
            bail!("FP16 linear input shape mismatch");
        }
        let w = fp16_bits(weight);
        let mut out = vec![0.0_f32; shape.rows * shape.out_features];
        // SAFETY: lengths checked above.
        self.check(unsafe {
            sys::ullis_cuda_fp16_linear(
                self.raw,
                input.as_ptr(),
                w.as_ptr(),
                out.as_mut_ptr(),
                shape.rows,
                shape.in_features,
                shape.out_features,
            )
        })?;
        Ok(out)
    }

    /// Forward half of `MetalRuntime::streamed_cross_entropy_fp16` (`src/metal.rs:2921`) with the
    /// head bias of the CPU model and an explicit `ignore_id` (`apply_head_ce`,
    /// `src/model.rs:3205-3228`): the `[rows, vocab]` logits never exist.
    #[allow(clippy::too_many_arguments)]
    pub fn streamed_cross_entropy_fp16(
        &self,
        hidden: &[f32],
        head: PackedLinearRef<'_>,
        labels: &[u32],
        ignore_id: u32,
        rows: usize,
        time: usize,
        channels: usize,
        vocab: usize,
    ) -> Result<StreamedCrossEntropy> {
        if hidden.len() != rows * channels
            || head.bits.len() != (channels * vocab).div_ceil(32)
            || head.scale.len() != vocab
            || head.bias.is_some_and(|b| b.len() != vocab)
            || labels.len() != rows
        {
            bail!("streamed CE input shape mismatch");
        }
        let mut row_loss = vec![0.0_f32; rows];
        let (mut mean_loss, mut n_valid) = (0.0_f32, 0_u64);
        // SAFETY: lengths checked above; the two scalars are valid out-pointers.
        self.check(unsafe {
            sys::ullis_cuda_streamed_ce(
                self.raw,
                hidden.as_ptr(),
                head.bits.as_ptr(),
                head.scale.as_ptr(),
                opt_ptr(head.bias),
                labels.as_ptr(),
                ignore_id,
                rows,
                time,
                channels,
                vocab,
                row_loss.as_mut_ptr(),
                &mut mean_loss,
                &mut n_valid,
            )
        })?;
        Ok(StreamedCrossEntropy { mean_loss, n_valid, row_loss })
    }

    /// `MetalRuntime::apply_latent_sgd` (`src/metal.rs:3006`): BinaryConnect step on
    /// `gradient * ste_scale`, then the re-packed sign words.
    pub fn apply_latent_sgd(
        &self,
        latent: &[u16],
        residual: &[f32],
        gradient: &[f32],
        learning_rate: f32,
        ste_scale: f32,
    ) -> Result<(Vec<u16>, Vec<f32>, Vec<u32>)> {
        let n = latent.len();
        if residual.len() != n || gradient.len() != n {
            bail!("latent SGD length mismatch");
        }
        let mut next_latent = vec![0_u16; n];
        let mut next_residual = vec![0.0_f32; n];
        let mut next_bits = vec![0_u32; n.div_ceil(32)];
        if n == 0 {
            return Ok((next_latent, next_residual, next_bits));
        }
        // SAFETY: all buffers hold n elements (ceil(n / 32) words for the bits).
        self.check(unsafe {
            sys::ullis_cuda_apply_latent_sgd(
                self.raw,
                latent.as_ptr(),
                residual.as_ptr(),
                gradient.as_ptr(),
                learning_rate,
                ste_scale,
                n,
                next_latent.as_mut_ptr(),
                next_residual.as_mut_ptr(),
                next_bits.as_mut_ptr(),
            )
        })?;
        Ok((next_latent, next_residual, next_bits))
    }

    /// `MetalRuntime::clipped_sgd_fp16` (`src/metal.rs:3053`): bit-identical to
    /// `Fp16Storage::apply_clipped_sgd` (`src/precision.rs:106-113`).
    pub fn clipped_sgd_fp16(
        &self,
        parameters: &[u16],
        residual: &[f32],
        gradient: &[f32],
        learning_rate: f32,
    ) -> Result<(Vec<u16>, Vec<f32>)> {
        self.sgd_fp16(parameters, residual, gradient, learning_rate, false)
    }

    /// `MetalRuntime::binaryconnect_sgd_fp16` (`src/metal.rs:3069`): bit-identical to
    /// `Fp16Storage::apply_binaryconnect_sgd` (`src/precision.rs:124-134`).
    pub fn binaryconnect_sgd_fp16(
        &self,
        parameters: &[u16],
        residual: &[f32],
        gradient: &[f32],
        learning_rate: f32,
    ) -> Result<(Vec<u16>, Vec<f32>)> {
        self.sgd_fp16(parameters, residual, gradient, learning_rate, true)
    }

    fn sgd_fp16(
        &self,
        parameters: &[u16],
        residual: &[f32],
        gradient: &[f32],
        learning_rate: f32,
        binaryconnect: bool,
    ) -> Result<(Vec<u16>, Vec<f32>)> {
        let n = parameters.len();
        if residual.len() != n || gradient.len() != n {
            bail!("FP16 SGD length mismatch");
        }
        let mut next = vec![0_u16; n];
        let mut next_residual = vec![0.0_f32; n];
        if n == 0 {
            return Ok((next, next_residual));
        }
        // SAFETY: five buffers of n elements each.
        let rc = unsafe {
            if binaryconnect {
                sys::ullis_cuda_binaryconnect_sgd_fp16(
                    self.raw,
                    parameters.as_ptr(),
                    residual.as_ptr(),
                    gradient.as_ptr(),
                    learning_rate,
                    n,
                    next.as_mut_ptr(),
                    next_residual.as_mut_ptr(),
                )
            } else {
                sys::ullis_cuda_clipped_sgd_fp16(
                    self.raw,
                    parameters.as_ptr(),
                    residual.as_ptr(),
                    gradient.as_ptr(),
                    learning_rate,
                    n,
                    next.as_mut_ptr(),
                    next_residual.as_mut_ptr(),
                )
            }
        };
        self.check(rc)?;
        Ok((next, next_residual))
    }

    /// Joins a data-parallel group of `world` processes (one per GPU).  `unique_id` comes from
    /// `dp_unique_id()` on rank 0 and reaches the other ranks by whatever channel the launcher has.
    pub fn dp_init(&self, rank: i32, world: i32, unique_id: &[u8; 128]) -> Result<()> {
        // SAFETY: `unique_id` is exactly the 128 bytes the call reads.
        self.check(unsafe { sys::ullis_cuda_dp_init(self.raw, rank, world, unique_id.as_ptr()) })
    }

    pub fn dp_finalize(&self) -> Result<()> {
        // SAFETY: live handle.
        self.check(unsafe { sys::ullis_cuda_dp_finalize(self.raw) })
    }
}

impl Drop for CudaRuntime {
    fn drop(&mut self) {
        // SAFETY: `raw` came from ullis_cuda_runtime_create and is destroyed exactly once.
        unsafe { sys::ullis_cuda_runtime_destroy(self.raw) };
    }
}

/// A fresh NCCL unique id (rank 0 creates it, every rank passes it to `CudaRuntime::dp_init`).
pub fn dp_unique_id() -> Result<[u8; 128]> {
    let mut id = [0_u8; 128];
    // SAFETY: `id` is the 128-byte buffer the call fills.
    let rc = unsafe { sys::ullis_cuda_dp_unique_id(id.as_mut_ptr()) };
    if rc != sys::ULLIS_CUDA_OK {
        bail!("{}", last_error(ptr::null()));
    }
    Ok(id)
}

/// The Heron model resident on the device: weights from the run's `checkpoint.safetensors`
/// (`ModelCheckpoint::to_safetensors_bytes`, `src/model.rs:3426-3468`), activations and automaton
/// state in HBM, one call per step.
#[derive(Debug)]
pub struct CudaHeron<'rt> {
    raw: *mut sys::ullis_cuda_model,
    rt: &'rt CudaRuntime,
}

impl<'rt> CudaHeron<'rt> {
    /// `UllisHeron::from_checkpoint` for the device (`from_safetensors_bytes`, `src/model.rs:3470-3553`):
    /// rejects format version 1, missing metadata and tensors whose shape contradicts the config.
    pub fn from_safetensors(rt: &'rt CudaRuntime, bytes: &[u8]) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: `bytes` is readable for its length; `raw` is a valid out-pointer.
        rt.check(unsafe { sys::ullis_cuda_model_load_safetensors(rt.raw, bytes.as_ptr(), bytes.len(), &mut raw) })?;
        Ok(Self { raw, rt })
    }

    /// `[d_model, n_layers, vocab_size, context_len, batch_size, dim_ffn]`.
    pub fn dims(&self) -> Result<[usize; 6]> {
        let mut dims = [0_usize; 6];
        // SAFETY: `dims` holds the six values the call writes.
        self.rt.check(unsafe { sys::ullis_cuda_model_dims(self.raw, dims.as_mut_ptr()) })?;
        Ok(dims)
    }

    /// Mean next-token cross-entropy and the number of supervised positions: the forward half of
    /// `train_step_on` (`src/model.rs:2865-2918`), `hidden` then `apply_head_ce`.
    pub fn forward_ce(&self, tokens: &[u32], labels: &[u32], ignore_id: u32, batch: usize, time: usize) -> Result<(f32, u64)> {
        if batch.checked_mul(time) != Some(tokens.len()) || labels.len() != tokens.len() {
            bail!("token shape or context length is invalid");
        }
        let (mut mean, mut sum, mut n) = (0.0_f32, 0.0_f64, 0_u64);
        // SAFETY: token and label lengths checked above; row_loss is not requested (null).
        self.rt.check(unsafe {
            sys::ullis_cuda_model_forward_ce(
                self.raw,
                tokens.as_ptr(),
                labels.as_ptr(),
                ignore_id,
                batch,
                time,
                &mut mean,
                &mut sum,
                &mut n,
                ptr::null_mut(),
            )
        })?;
        Ok((mean, n))
    }

    /// The same step for one rank of a data-parallel group: this rank's sequences in, the mean over
    /// EVERY rank's supervised positions out (sums and counts are added, not means;
    /// `src/model.rs:3253-3257`).
    pub fn forward_ce_global(&self, tokens: &[u32], labels: &[u32], ignore_id: u32, batch: usize, time: usize) -> Result<(f32, u64)> {
        if batch.checked_mul(time) != Some(tokens.len()) || labels.len() != tokens.len() {
            bail!("token shape or context length is invalid");
        }
        // SAFETY: lengths checked above.
        self.rt.check(unsafe {
            sys::ullis_cuda_model_upload_tokens(self.raw, tokens.as_ptr(), labels.as_ptr(), batch, time)
        })?;
        // SAFETY: live handle.
        self.rt.check(unsafe { sys::ullis_cuda_model_enqueue_forward_ce(self.raw, ignore_id, batch, time) })?;
        let (mut mean, mut sum, mut n) = (0.0_f32, 0.0_f64, 0_u64);
        // SAFETY: three valid out-pointers.
        self.rt.check(unsafe { sys::ullis_cuda_model_read_loss_global(self.raw, &mut mean, &mut sum, &mut n) })?;
        Ok((mean, n))
    }

    /// `UllisHeron::logits` (`src/model.rs:2685-2688`): `[batch * time, vocab]`.
    pub fn logits(&self, tokens: &[u32], batch: usize, time: usize) -> Result<Vec<f32>> {
        if batch.checked_mul(time) != Some(tokens.len()) {
            bail!("token shape or context length is invalid");
        }
        let vocab = self.dims()?[2];
        let mut logits = vec![0.0_f32; tokens.len() * vocab];
        // SAFETY: `logits` holds batch * time * vocab floats.
        self.rt.check(unsafe { sys::ullis_cuda_model_logits(self.raw, tokens.as_ptr(), batch, time, logits.as_mut_ptr()) })?;
        Ok(logits)
    }

    /// `UllisHeron::hidden` (`src/model.rs:2644-2683`): `[batch * time, d_model]` after `ln_out`.
    pub fn hidden(&self, tokens: &[u32], batch: usize, time: usize) -> Result<Vec<f32>> {
        if batch.checked_mul(time) != Some(tokens.len()) {
            bail!("token shape or context length is invalid");
        }
        let d_model = self.dims()?[0];
        let mut hidden = vec![0.0_f32; tokens.len() * d_model];
        // SAFETY: `hidden` holds batch * time * d_model floats.
        self.rt.check(unsafe { sys::ullis_cuda_model_hidden(self.raw, tokens.as_ptr(), batch, time, hidden.as_mut_ptr()) })?;
        Ok(hidden)
    }

    /// `UllisHeron::generate_state` (`src/model.rs:2691-2715`) for `batch` conversations in lock step.
    pub fn generate_state(&self, batch: usize) -> Result<CudaGenerateState<'_, 'rt>> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer.
        self.rt.check(unsafe { sys::ullis_cuda_generate_state_create(self.raw, batch, &mut raw) })?;
        Ok(CudaGenerateState { raw, model: self, batch })
    }

    /// Optimiser state on the device (`train_step_on`, `src/model.rs:2827-3020`, stop_grad_bits).
    /// `checkpoint` restores the `.latent` / `.residual` carry of a resumed run.
    pub fn train_state(&self, checkpoint: Option<&[u8]>) -> Result<CudaTrainState<'_, 'rt>> {
        let mut raw = ptr::null_mut();
        let (p, len) = checkpoint.map_or((ptr::null(), 0), |b| (b.as_ptr(), b.len()));
        // SAFETY: `p` is null or readable for `len` bytes.
        self.rt.check(unsafe { sys::ullis_cuda_train_state_create(self.raw, p, len, &mut raw) })?;
        Ok(CudaTrainState { raw, model: self })
    }
}

impl Drop for CudaHeron<'_> {
    fn drop(&mut self) {
        // SAFETY: `raw` came from ullis_cuda_model_load_safetensors and is destroyed exactly once,
        // before the runtime it borrows.
        unsafe { sys::ullis_cuda_model_destroy(self.raw) };
    }
}

/// `HeronGenerateState` (`src/model.rs:2433-2454`) with the automata on the device.
#[derive(Debug)]
pub struct CudaGenerateState<'m, 'rt> {
    raw: *mut sys::ullis_cuda_generate_state,
    model: &'m CudaHeron<'rt>,
    batch: usize,
}

impl CudaGenerateState<'_, '_> {
    /// `HeronGenerateState::time` (`src/model.rs:2449-2453`).
    pub fn time(&self) -> usize {
        // SAFETY: live handle.
        unsafe { sys::ullis_cuda_generate_state_time(self.raw) }
    }

    /// Back to an empty context without reallocating (`RosaSam::reset`, `src/rosa.rs:66-74`).
    pub fn reset(&mut self) -> Result<()> {
        // SAFETY: live handle.
        self.model.rt.check(unsafe { sys::ullis_cuda_generate_state_reset(self.raw) })
    }

    /// `UllisHeron::generate_step` (`src/model.rs:2717-2753`): one token per conversation in, the
    /// last-position logits `[batch, vocab]` out.
    pub fn step(&mut self, tokens: &[u32]) -> Result<Vec<f32>> {
        if tokens.len() != self.batch {
            bail!("generate_step takes one token per sequence");
        }
        let vocab = self.model.dims()?[2];
        let mut logits = vec![0.0_f32; self.batch * vocab];
        // SAFETY: `tokens` holds `batch` ids, `logits` batch * vocab floats.
        self.model
            .rt
            .check(unsafe { sys::ullis_cuda_generate_step(self.raw, tokens.as_ptr(), logits.as_mut_ptr()) })?;
        Ok(logits)
    }
}

impl Drop for CudaGenerateState<'_, '_> {
    fn drop(&mut self) {
        // SAFETY: destroyed exactly once, before the model it borrows.
        unsafe { sys::ullis_cuda_generate_state_destroy(self.raw) };
    }
}

/// `streams` independent `RosaSam` automata (`src/rosa.rs:55-176`) kept on the device between calls: the
/// per-layer state of a generate state at op level.
#[derive(Debug)]
pub struct CudaRosaPushers<'rt> {
    raw: *mut sys::ullis_cuda_rosa_pushers,
    rt: &'rt CudaRuntime,
    streams: usize,
}

impl<'rt> CudaRosaPushers<'rt> {
    /// `RosaSam::new` for every stream; `capacity` pushes fit (the reference's vectors grow instead).
    pub fn new(rt: &'rt CudaRuntime, streams: usize, capacity: usize) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        // SAFETY: `raw` receives a fresh handle or stays null.
        rt.check(unsafe { sys::ullis_cuda_rosa_pushers_create(rt.raw, streams, capacity, &mut raw) })?;
        Ok(Self { raw, rt, streams })
    }

    /// `RosaSam::reset` (`src/rosa.rs:66-74`).
    pub fn reset(&mut self) -> Result<()> {
        // SAFETY: live handle.
        self.rt.check(unsafe { sys::ullis_cuda_rosa_pushers_reset(self.raw) })
    }

    /// `RosaSam::push` (`src/rosa.rs:100-176`) for every stream, once per row: `q`, `k`, `v` are
    /// `[steps, streams]` of 0 / 1; returns idx in the same layout.
    pub fn push(&mut self, q: &[u8], k: &[u8], v: &[u8]) -> Result<Vec<u8>> {
        if self.streams == 0 || q.len() % self.streams != 0 || k.len() != q.len() || v.len() != q.len() {
            bail!("ROSA pushers take [steps, streams] bits for q, k and v");
        }
        let steps = q.len() / self.streams;
        let mut idx = vec![0_u8; q.len()];
        // SAFETY: the four slices hold steps * streams bytes.
        self.rt.check(unsafe {
            sys::ullis_cuda_rosa_pushers_push(self.raw, q.as_ptr(), k.as_ptr(), v.as_ptr(), steps, idx.as_mut_ptr())
        })?;
        Ok(idx)
    }
}

impl Drop for CudaRosaPushers<'_> {
    fn drop(&mut self) {
        // SAFETY: destroyed exactly once, before the runtime it borrows.
        unsafe { sys::ullis_cuda_rosa_pushers_destroy(self.raw) };
    }
}

/// The fields of `CausalLoss` a device step produces (`src/model.rs:60-83`).
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct CudaTrainStep {
    pub next_token: f32,
    pub next_token_count: u64,
    pub flips_head: u64,
    pub flips_cmix: u64,
    pub flips_rosa_o: u64,
}

/// Latents and FP32 carry of the trained tensors, on the device.
#[derive(Debug)]
pub struct CudaTrainState<'m, 'rt> {
    raw: *mut sys::ullis_cuda_train_state,
    model: &'m CudaHeron<'rt>,
}

impl CudaTrainState<'_, '_> {
    /// `UllisHeron::train_step_with_labels` (`src/model.rs:2773-2785`).
    pub fn train_step(
        &mut self,
        tokens: &[u32],
        labels: &[u32],
        ignore_id: u32,
        batch: usize,
        time: usize,
        learning_rate: f32,
    ) -> Result<CudaTrainStep> {
        if batch.checked_mul(time) != Some(tokens.len()) || labels.len() != tokens.len() {
            bail!("token shape or context length is invalid");
        }
        let mut r = sys::ullis_cuda_train_result::default();
        // SAFETY: lengths checked above; `r` is a valid out-pointer.
        self.model.rt.check(unsafe {
            sys::ullis_cuda_model_train_step(
                self.raw,
                tokens.as_ptr(),
                labels.as_ptr(),
                ignore_id,
                batch,
                time,
                learning_rate,
                &mut r,
            )
        })?;
        Ok(CudaTrainStep {
            next_token: r.mean_loss,
            next_token_count: r.n_valid,
            flips_head: r.flips_head,
            flips_cmix: r.flips_cmix,
            flips_rosa_o: r.flips_rosa_o,
        })
    }

    /// Reads one tensor of the trained model or of its carry back by checkpoint name
    /// (`"head.bits"`, `"blocks.0.rosa.o.latent"`, `"embedding.residual"`, ...).
    pub fn read_bytes(&self, name: &str, bytes: usize) -> Result<Vec<u8>> {
        let c_name = std::ffi::CString::new(name)?;
        let mut out = vec![0_u8; bytes];
        // SAFETY: `out` holds `bytes` writable bytes; `c_name` is NUL-terminated.
        self.model.rt.check(unsafe {
            sys::ullis_cuda_train_state_read(self.raw, c_name.as_ptr(), out.as_mut_ptr().cast(), bytes)
        })?;
        Ok(out)
    }

    /// `UllisHeron::install_head_unigram_prior` (`src/model.rs:3034-3110`).
    pub fn install_head_unigram_prior(&mut self, labels: &[u32], ignore_id: u32) -> Result<sys::ullis_cuda_head_unigram_install> {
        let mut r = sys::ullis_cuda_head_unigram_install::default();
        // SAFETY: `labels` is readable for its length; `r` is a valid out-pointer.
        self.model.rt.check(unsafe {
            sys::ullis_cuda_train_state_install_head_unigram_prior(self.raw, labels.as_ptr(), labels.len(), ignore_id, &mut r)
        })?;
        Ok(r)
    }
}

impl Drop for CudaTrainState<'_, '_> {
    fn drop(&mut self) {
        // SAFETY: destroyed exactly once, before the model it borrows.
        unsafe { sys::ullis_cuda_train_state_destroy(self.raw) };
    }
}
