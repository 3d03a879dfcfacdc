//! B200 (sm_100a) kernels of the quantized projection path behind the operator types the
//! engine already calls on `tuisko-kernels-sm120` / `tuisko-kernels-sm89`: the same type names,
//! method names and argument order, forwarding to the C ABI of `libtuisko_sm100`
//! (`include/tuisko_sm100.h`, declared in `tuisko_gpu::ffi_sm100`).
//!
//! Differences from the sm_120 crate, all visible here:
//! * one shared [`Sm100Context`] replaces the per-operator module load (`*Op::new` takes it);
//!   creating it is the only place the library allocates device memory;
//! * any `1 ..= max_rows` row count is admitted, not only the exact routes `1..=8` and 16;
//! * planes read through TMA (activation / weight codes) must be 128-byte aligned;
//! * the NVFP4 operators take the activation code / scale planes and the checkpoint's
//!   `input_global_scale` divisor as well (the contraction runs W4A4 on `tcgen05`).
//!
//! This crate has NOT been compiled: the image the CUDA library was built and tested in has no
//! Rust toolchain.  The tested binding of the same ABI is the `ctypes` mirror
//! (`tuiskollm_b200/_lib.py`, `tuiskollm_b200/ops.py`).
#![allow(clippy::too_many_arguments, clippy::missing_safety_doc)]

use std::ffi::CStr;
use std::marker::PhantomData;
use std::ptr;
use std::sync::Arc;

use cuda_core::{CudaContext, CudaStream};
use tuisko_gpu::ffi_sm100 as ffi;
use tuisko_gpu::{GpuError, GpuResult};
use tuisko_model::{Arch, Qwen38_27B};

mod private {
    pub trait Sealed {}
    impl Sealed for tuisko_model::Qwen38_27B {}
}

/// Model architecture admitted by the sm_100a library (run-time geometry, checked at create).
pub trait Sm100Arch: Arch + private::Sealed {}
impl Sm100Arch for Qwen38_27B {}

/// Largest row count any launch passes (decode batches and prefill chunks).
pub const MAX_ROWS: usize = 2048;

/// One `tk100_ctx`: kernel routes, split-K scratch, tile tickets and the device status word.
/// Create it with the engine's CUDA context bound to the calling thread
/// (`tuisko-gpu/src/arena.rs:123-128`); launch from one thread per context.
pub struct Sm100Context {
    raw: *mut ffi::Tk100Ctx,
    _cuda: Arc<CudaContext>,
}

// SAFETY: the C context is used by one launching thread at a time (`&self` methods are called
// serially during graph capture, tuisko-engine/src/dense_fp8_mlp.rs:385-402).
unsafe impl Send for Sm100Context {}

impl Sm100Context {
    /// `tk100_create` for architecture `A` on the device of `context`.
    pub fn new<A: Sm100Arch>(context: &Arc<CudaContext>, device: i32) -> GpuResult<Arc<Self>> {
        let config = ffi::Tk100Config {
            abi_version: ffi::TK100_ABI_VERSION,
            device,
            hidden: A::HIDDEN as u32,
            intermediate: A::INTERMEDIATE as u32,
            rms_norm_epsilon: A::RMS_NORM_EPSILON,
            max_rows: MAX_ROWS as u32,
            workspace_bytes: 0,
        };
        let mut raw = ptr::null_mut();
        // SAFETY: `config` and `raw` are valid for the call.
        let status = unsafe { ffi::tk100_create(&config, &mut raw) };
        if status != 0 {
            return Err(error_from(status, ptr::null()));
        }
        Ok(Arc::new(Self { raw, _cuda: Arc::clone(context) }))
    }

    fn check(&self, status: ffi::Tk100Status) -> GpuResult<()> {
        if status == 0 { Ok(()) } else { Err(error_from(status, self.raw)) }
    }

    /// Reads and clears the device status word (`TK100_DEVICE_*` bits); synchronises `stream`.
    pub fn device_status(&self, stream: &CudaStream) -> GpuResult<u32> {
        let mut word = 0u32;
        // SAFETY: `word` outlives the synchronous call.
        self.check(unsafe { ffi::tk100_device_status(self.raw, stream.cu_stream().cast(), &mut word) })?;
        Ok(word)
    }

    /// Encodes the TMA tensor map of a weight-code plane at load time (`tk100_register_plane`);
    /// the counterpart of the sm_120 operators' route preparation in `*Op::new`.
    ///
    /// # Safety
    ///
    /// `weight_codes` is a live device plane of `rows * row_bytes` bytes, 128-byte aligned.
    pub unsafe fn register_plane(&self, weight_codes: *const u8, rows: usize, row_bytes: usize) -> GpuResult<()> {
        self.check(unsafe {
            ffi::tk100_register_plane(self.raw, weight_codes.cast(), rows as u64, row_bytes as u64)
        })
    }
}

impl Drop for Sm100Context {
    fn drop(&mut self) {
        // SAFETY: `raw` came from tk100_create and is dropped once.
        unsafe { ffi::tk100_destroy(self.raw) }
    }
}

/// Maps `tk100_status` 1..=6 onto `GpuErrorCode` (`tuisko-gpu/src/error.rs:8-43`); the library's
/// message already carries the `[gpu.*]` prefix.  `GpuError::{driver,arena,graph,context,module}_message`
/// are one-line public constructors to add to `tuisko-gpu/src/error.rs` beside `invalid_launch`
/// (the existing ones, `error.rs:97-124`, are `pub(crate)` and take typed sources).
fn error_from(status: ffi::Tk100Status, ctx: *const ffi::Tk100Ctx) -> GpuError {
    // SAFETY: tk100_last_error returns a NUL-terminated string owned by the library.
    let message = unsafe { CStr::from_ptr(ffi::tk100_last_error(ctx)) }.to_string_lossy().into_owned();
    match status {
        2 => GpuError::arena_message(message),
        3 => GpuError::graph_message(message),
        4 => GpuError::context_message(message),
        5 => GpuError::invalid_launch(message),
        6 => GpuError::module_message(message),
        _ => GpuError::driver_message(message),
    }
}

fn rows_i32(rows: usize) -> i32 {
    i32::try_from(rows).unwrap_or(i32::MAX) // out-of-range counts are rejected by the library
}

/// `ResidualNormOp` (`tuisko-kernels-sm120/src/residual_norm.rs:382-508`).
pub struct ResidualNormOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> ResidualNormOp<A> {
    /// Replaces the module load of `residual_norm.rs:396-416`.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// `launch_plain` (`residual_norm.rs:425-456`).
    pub unsafe fn launch_plain(
        &self, stream: &CudaStream, batch: usize, input: *const u16, weight: *const u16,
        output: *mut u16,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_rms_norm(self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), input, weight, output)
        })
    }

    /// `launch_residual` (`residual_norm.rs:467-507`).
    pub unsafe fn launch_residual(
        &self, stream: &CudaStream, batch: usize, residual_input: *const u16, branch: *const u16,
        weight: *const u16, residual_output: *mut u16, normalized_output: *mut u16,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_residual_rms_norm(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), residual_input, branch,
                weight, residual_output, normalized_output,
            )
        })
    }

    /// The fused producer: `launch_residual` (or `launch_plain` with `branch == null`) plus the
    /// per-token E4M3 quantiser of the next projection, one kernel.  The projection is then
    /// launched with `input == null`.
    pub unsafe fn launch_quantize(
        &self, stream: &CudaStream, batch: usize, residual_input: *const u16, branch: *const u16,
        weight: *const u16, residual_output: *mut u16, normalized_output: *mut u16,
        activation_codes: *mut u8, activation_scales: *mut f32,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_residual_rms_norm_quantize(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), residual_input, branch,
                weight, residual_output, normalized_output, activation_codes, activation_scales,
            )
        })
    }

    /// The fused producer with the NVFP4 form of the normalised row as well (for the W4A4 MLP).
    pub unsafe fn launch_quantize_nvfp4(
        &self, stream: &CudaStream, batch: usize, residual_input: *const u16, branch: *const u16,
        weight: *const u16, residual_output: *mut u16, normalized_output: *mut u16,
        activation_codes: *mut u8, activation_scales: *mut f32, input_global_divisor: f32,
        nvfp4_codes: *mut u8, nvfp4_scales: *mut u8,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_residual_rms_norm_quantize_nvfp4(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), residual_input, branch,
                weight, residual_output, normalized_output, activation_codes, activation_scales,
                input_global_divisor, nvfp4_codes, nvfp4_scales,
            )
        })
    }
}

macro_rules! fp8_projection_op {
    ($(#[$doc:meta])* $name:ident, $entry:ident, $rows:expr) => {
        $(#[$doc])*
        pub struct $name<A: Sm100Arch = Qwen38_27B> {
            ctx: Arc<Sm100Context>,
            _arch: PhantomData<A>,
        }

        impl<A: Sm100Arch> $name<A> {
            /// Replaces the module load and route preparation of the sm_120 operator.
            pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
                Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
            }

            /// Same argument order as the sm_120 `launch`
            /// (`tuisko-kernels-sm120/src/fp8/projection.rs:557-567`).  `input == null`: the
            /// activation planes already hold the fused producer's codes and scales.
            pub unsafe fn launch(
                &self, stream: &CudaStream, rows: usize, input: *const u16,
                activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
                weight_scales: *const u16, output: *mut u16,
            ) -> GpuResult<()> {
                let out_rows: usize = $rows;
                self.ctx.check(unsafe {
                    ffi::$entry(
                        self.ctx.raw, stream.cu_stream().cast(), rows_i32(rows), out_rows as i32,
                        input, activation_codes, activation_scales, weight_codes, weight_scales,
                        output,
                    )
                })
            }
        }
    };
}

fp8_projection_op!(
    /// `FullAttentionQkvOp` (`tuisko-kernels-sm120/src/fp8/projection.rs:510-611`).
    FullAttentionQkvOp, tk100_fp8_qkv, A::ATTENTION_QKV_ROWS
);
fp8_projection_op!(
    /// `GdnInputProjectionOp` (`tuisko-kernels-sm120/src/fp8/projection.rs:613-702`).
    GdnInputProjectionOp, tk100_fp8_gdn_input, A::GDN_INPUT_ROWS
);

/// `GdnOutputProjectionOp` (`tuisko-kernels-sm120/src/fp8/gdn_output.rs:178`): reduction length
/// `GDN_VALUE_ROWS`, `HIDDEN` output rows.
pub struct GdnOutputProjectionOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> GdnOutputProjectionOp<A> {
    /// Replaces the module load of the sm_120 operator.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// Same argument order as the sm_120 `launch`.
    pub unsafe fn launch(
        &self, stream: &CudaStream, rows: usize, input: *const u16, activation_codes: *mut u8,
        activation_scales: *mut f32, weight_codes: *const u8, weight_scales: *const u16,
        output: *mut u16,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_fp8_gdn_output(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(rows), A::GDN_VALUE_ROWS as i32,
                input, activation_codes, activation_scales, weight_codes, weight_scales, output,
            )
        })
    }
}

/// Device counterpart of `tuisko-model/src/materialize.rs`: the fused QKV gather
/// (`gather_source_planes`, `:295-314`) and the NVFP4 block-scale permutation
/// (`swizzle_scale_planes`, `:353-408`) on planes that were uploaded as the checkpoint stores them.
pub struct MaterializeOp {
    ctx: Arc<Sm100Context>,
}

impl MaterializeOp {
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx) })
    }

    /// Concatenates up to three device planes (`(address, bytes)` pairs) into `output`.
    pub unsafe fn gather(
        &self, stream: &CudaStream, planes: &[(*const u8, u64)], output: *mut u8,
    ) -> GpuResult<()> {
        let sources = planes.iter().map(|plane| plane.0.cast()).collect::<Vec<*const std::ffi::c_void>>();
        let bytes = planes.iter().map(|plane| plane.1).collect::<Vec<u64>>();
        self.ctx.check(unsafe {
            ffi::tk100_materialize_gather(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(planes.len()), sources.as_ptr(),
                bytes.as_ptr(), output.cast(),
            )
        })
    }

    /// One (down) or two (gate, up) row-major `[rows_per_plane, groups_per_row]` E4M3 planes
    /// into the `BlockScaleK16M128x4` order.
    pub unsafe fn swizzle_scales(
        &self, stream: &CudaStream, planes: &[*const u8], rows_per_plane: usize,
        groups_per_row: usize, output: *mut u8,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_materialize_nvfp4_scales(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(planes.len()), planes.as_ptr(),
                rows_per_plane as u64, groups_per_row as u64, output,
            )
        })
    }
}

/// Device counterpart of the engine's host `Sampler` (`tuisko-engine/src/sampling.rs:56-101`)
/// for a decode batch: the BF16 logit rows stay in device memory, one launch selects every
/// request's token.  The caller owns the generator states (`[rows]` u64, started from
/// [`DeviceSamplerOp::initial_state`]), the scratch ([`DeviceSamplerOp::scratch_bytes`], zeroed
/// once) and the decision plane.
pub struct DeviceSamplerOp {
    ctx: Arc<Sm100Context>,
}

impl DeviceSamplerOp {
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx) })
    }

    /// `XorShift64::new` (`sampling.rs:247-250`).
    pub fn initial_state(seed: u64) -> u64 {
        unsafe { ffi::tk100_sampler_initial_state(seed) }
    }

    pub fn scratch_bytes(rows: usize, vocab: usize) -> usize {
        unsafe { ffi::tk100_sampler_scratch_bytes(rows_i32(rows), vocab as i32) }
    }

    /// `options` holds one entry per request and is validated with the reference's rules
    /// before the launch; `top_out` may be null.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn launch(
        &self, stream: &CudaStream, vocab: usize, logits: *const u16,
        options: &[ffi::Tk100SamplingOptions], rng_state: *mut u64, scratch: *mut u64,
        decisions: *mut ffi::Tk100SampleDecision, top_out: *mut u32,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_sample(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(options.len()), vocab as i32,
                logits, options.as_ptr(), rng_state, scratch, decisions, top_out,
            )
        })
    }
}

/// `GdnPrepareOp` (`tuisko-kernels-sm120/src/gdn/prepare.rs:176-290`): control mat-vecs and the
/// width-4 causal convolution of a decode batch of 1..=8 tokens, one launch.
pub struct GdnPrepareOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> GdnPrepareOp<A> {
    /// Replaces the module load and the eight prepared routes of the sm_120 operator.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// Same argument order and safety contract as the sm_120 `launch`.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn launch(
        &self, stream: &CudaStream, batch: usize, input: *const u16, control_weights: *const u16,
        a_log: *const u16, dt_bias: *const u16, projected: *const u16,
        convolution_weights: *const u16, state_rows: *const u32, history: *mut u16,
        log_decay: *mut f32, beta: *mut f32, convolved: *mut u16,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_gdn_prepare(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), input, control_weights,
                a_log, dt_bias, projected, convolution_weights, state_rows, history, log_decay,
                beta, convolved,
            )
        })
    }
}

/// `GdnRecurrenceOp` (`tuisko-kernels-sm120/src/gdn/recurrence.rs:137-236`).
pub struct GdnRecurrenceOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> GdnRecurrenceOp<A> {
    /// Replaces the module load and the eight prepared routes of the sm_120 operator.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// Same argument order and safety contract as the sm_120 `launch`.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn launch(
        &self, stream: &CudaStream, batch: usize, qkv: *const u16, projected: *const u16,
        log_decay: *const f32, beta: *const f32, norm_weight: *const u16,
        state_rows: *const u32, state: *mut f32, output: *mut u16,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_gdn_recurrence(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), qkv, projected,
                log_decay, beta, norm_weight, state_rows, state, output,
            )
        })
    }
}

macro_rules! fp8_mlp_op {
    ($(#[$doc:meta])* $name:ident, $entry:ident) => {
        $(#[$doc])*
        pub struct $name<A: Sm100Arch = Qwen38_27B> {
            ctx: Arc<Sm100Context>,
            _arch: PhantomData<A>,
        }

        impl<A: Sm100Arch> $name<A> {
            /// Replaces the module load and route preparation of the sm_120 operator.
            pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
                Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
            }

            /// Same argument order as the sm_120 `launch`.
            pub unsafe fn launch(
                &self, stream: &CudaStream, rows: usize, input: *const u16,
                activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
                weight_scales: *const u16, output: *mut u16,
            ) -> GpuResult<()> {
                self.ctx.check(unsafe {
                    ffi::$entry(
                        self.ctx.raw, stream.cu_stream().cast(), rows_i32(rows), input,
                        activation_codes, activation_scales, weight_codes, weight_scales, output,
                    )
                })
            }
        }
    };
}

fp8_mlp_op!(
    /// `DenseFp8SwiGluOp` (`tuisko-kernels-sm120/src/fp8/swiglu.rs:366-376`): gate/up + SwiGLU.
    DenseFp8SwiGluOp, tk100_fp8_swiglu
);
fp8_mlp_op!(
    /// `DenseFp8DownOp` (`tuisko-kernels-sm120/src/fp8/down.rs:197-207`).
    DenseFp8DownOp, tk100_fp8_down
);

/// `LmHeadOp` (`tuisko-kernels-sm120/src/fp8/projection.rs:704-793`) with the greedy selection of
/// `tuisko-engine/src/sampling.rs:162-173` folded into the kernel.
pub struct LmHeadOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    vocab_rows: usize,
    vocab_offset: usize,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> LmHeadOp<A> {
    /// The whole vocabulary on one GPU.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Self::sharded(ctx, A::VOCAB, 0)
    }

    /// One rank's contiguous shard `[vocab_offset, vocab_offset + vocab_rows)`.
    pub fn sharded(ctx: &Arc<Sm100Context>, vocab_rows: usize, vocab_offset: usize) -> GpuResult<Self> {
        if vocab_rows == 0 || vocab_rows % 16 != 0 || vocab_offset + vocab_rows > A::VOCAB {
            return Err(GpuError::invalid_launch(format!(
                "LM head shard [{vocab_offset}, {}) is not a multiple of 16 rows inside the vocabulary",
                vocab_offset + vocab_rows
            )));
        }
        Ok(Self { ctx: Arc::clone(ctx), vocab_rows, vocab_offset, _arch: PhantomData })
    }

    /// The reference's signature (`projection.rs:751-761`): BF16 logits only.
    pub unsafe fn launch(
        &self, stream: &CudaStream, batch: usize, input: *const u16, activation_codes: *mut u8,
        activation_scales: *mut f32, weight_codes: *const u8, weight_scales: *const u16,
        output: *mut u16,
    ) -> GpuResult<()> {
        unsafe {
            self.launch_greedy(
                stream, batch, input, activation_codes, activation_scales, weight_codes,
                weight_scales, output, ptr::null_mut(), ptr::null_mut(), ptr::null_mut(),
            )
        }
    }

    /// With the optional fp32 logits plane and the fused argmax (`argmax_scratch`: one zeroed u64
    /// per row from the arena; `pairs`: `(max, global index)` per row).
    pub unsafe fn launch_greedy(
        &self, stream: &CudaStream, batch: usize, input: *const u16, activation_codes: *mut u8,
        activation_scales: *mut f32, weight_codes: *const u8, weight_scales: *const u16,
        output: *mut u16, logits_f32: *mut f32, argmax_scratch: *mut u64,
        pairs: *mut ffi::Tk100ArgmaxPair,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_fp8_lm_head(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), self.vocab_rows as i32,
                self.vocab_offset as i32, input, activation_codes, activation_scales, weight_codes,
                weight_scales, output, logits_f32, argmax_scratch, pairs,
            )
        })
    }

    /// One rank of the sharded LM head in ONE launch: projection, per-shard argmax, peer-store
    /// exchange over NVLink and merge (`peer_buffers` empty when `world == 1`).
    pub unsafe fn launch_sharded(
        &self, stream: &CudaStream, batch: usize, input: *const u16, activation_codes: *mut u8,
        activation_scales: *mut f32, weight_codes: *const u8, weight_scales: *const u16,
        output: *mut u16, logits_f32: *mut f32, argmax_scratch: *mut u64, world: usize, rank: usize,
        peer_buffers: &[u64], merged_pairs: *mut ffi::Tk100ArgmaxPair,
    ) -> GpuResult<()> {
        if world > 1 && peer_buffers.len() != world {
            return Err(GpuError::invalid_launch("sharded LM head needs one peer buffer per rank"));
        }
        let peers = if peer_buffers.is_empty() { ptr::null() } else { peer_buffers.as_ptr() };
        self.ctx.check(unsafe {
            ffi::tk100_fp8_lm_head_sharded(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), self.vocab_rows as i32,
                self.vocab_offset as i32, input, activation_codes, activation_scales, weight_codes,
                weight_scales, output, logits_f32, argmax_scratch, world as i32, rank as i32, peers,
                merged_pairs,
            )
        })
    }

    /// Vocabulary shards: peer-store exchange of the per-shard maxima fused with the merge
    /// (after `launch_greedy` with `pairs == null`).
    pub unsafe fn exchange(
        &self, stream: &CudaStream, batch: usize, world: usize, rank: usize,
        argmax_scratch: *mut u64, peer_buffers: &[u64], output: *mut ffi::Tk100ArgmaxPair,
    ) -> GpuResult<()> {
        if peer_buffers.len() != world {
            return Err(GpuError::invalid_launch("argmax exchange needs one peer buffer per rank"));
        }
        self.ctx.check(unsafe {
            ffi::tk100_argmax_exchange(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), world as i32, rank as i32,
                argmax_scratch, peer_buffers.as_ptr(), output,
            )
        })
    }
}

/// `Nvfp4SwiGluOp` (`tuisko-kernels-sm89/src/nvfp4/swiglu.rs:470-571`).
pub struct Nvfp4SwiGluOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> Nvfp4SwiGluOp<A> {
    /// Replaces `Nvfp4SwiGluOp::new` (`nvfp4/swiglu.rs:495`).
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// The reference's arguments (`nvfp4/swiglu.rs:525-534`) followed by the W4A4 additions.
    pub unsafe fn launch(
        &self, stream: &CudaStream, batch: usize, input: *const u16, weight_codes: *const u8,
        weight_scales: *const u8, weight_scale_divisor: f32, output: *mut u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_nvfp4_gate_up_swiglu(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), input, activation_codes,
                activation_scales, input_global_divisor, weight_codes, weight_scales,
                weight_scale_divisor, output,
            )
        })
    }
}

/// `Nvfp4DownOp` (`tuisko-kernels-sm89/src/nvfp4/down.rs:455-556`).
pub struct Nvfp4DownOp<A: Sm100Arch = Qwen38_27B> {
    ctx: Arc<Sm100Context>,
    _arch: PhantomData<A>,
}

impl<A: Sm100Arch> Nvfp4DownOp<A> {
    /// Replaces `Nvfp4DownOp::new`.
    pub fn new(ctx: &Arc<Sm100Context>) -> GpuResult<Self> {
        Ok(Self { ctx: Arc::clone(ctx), _arch: PhantomData })
    }

    /// The reference's arguments (`nvfp4/down.rs:510-519`) followed by the W4A4 additions.
    pub unsafe fn launch(
        &self, stream: &CudaStream, batch: usize, input: *const u16, weight_codes: *const u8,
        weight_scales: *const u8, weight_scale_divisor: f32, output: *mut u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
    ) -> GpuResult<()> {
        self.ctx.check(unsafe {
            ffi::tk100_nvfp4_down(
                self.ctx.raw, stream.cu_stream().cast(), rows_i32(batch), input, activation_codes,
                activation_scales, input_global_divisor, weight_codes, weight_scales,
                weight_scale_divisor, output,
            )
        })
    }
}
