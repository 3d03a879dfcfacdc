//! `extern "C"` declarations of `libtuisko_sm100` (`include/tuisko_sm100.h`), one per exported
//! symbol, in the header's order.  Add `pub mod ffi_sm100;` to `tuisko-gpu/src/lib.rs`.
//!
//! NOT compiled in the image the library was built in (no Rust toolchain there); a CPU test of
//! the kernel repository checks that this file declares exactly the header's symbols.
#![allow(missing_docs, clippy::too_many_arguments)]

use std::ffi::{c_char, c_int, c_void};

/// `CUstream` / `cudaStream_t`.
pub type Tk100Stream = *mut c_void;

/// `tk100_status`: 0 ok, 1..=6 = `GpuErrorCode::{Driver, Arena, Graph, Context, Launch, Module}`.
pub type Tk100Status = c_int;

pub const TK100_ABI_VERSION: u32 = 1;
pub const TK100_DEVICE_WAIT_TIMEOUT: u32 = 1;
pub const TK100_DEVICE_NONFINITE_LOGIT: u32 = 2;
pub const TK100_DEVICE_NONFINITE_INPUT: u32 = 4;
pub const TK100_DEVICE_BAD_ARGUMENT: u32 = 8;
pub const TK100_STATIC_MAX_ROWS: c_int = 256;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct Tk100Config {
    pub abi_version: u32,
    pub device: i32,
    pub hidden: u32,
    pub intermediate: u32,
    pub rms_norm_epsilon: f32,
    pub max_rows: u32,
    pub workspace_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct Tk100ArgmaxPair {
    pub value: f32,
    pub index: i32,
}

/// `tk100_sampling_options`: one request's controls and stop-token pair.
#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Tk100SamplingOptions {
    pub temperature: f32,
    pub top_p: f32,
    pub top_k: u32,
    pub stop_ids: [u32; 2],
}

/// `tk100_sample_decision`.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default, Eq, PartialEq)]
pub struct Tk100SampleDecision {
    pub token_id: u32,
    pub stopped: u32,
}

#[repr(C)]
pub struct Tk100Ctx {
    _opaque: [u8; 0],
}

unsafe extern "C" {
    pub fn tk100_create(config: *const Tk100Config, out: *mut *mut Tk100Ctx) -> Tk100Status;
    pub fn tk100_destroy(ctx: *mut Tk100Ctx);
    pub fn tk100_last_error(ctx: *const Tk100Ctx) -> *const c_char;
    pub fn tk100_device_status(ctx: *mut Tk100Ctx, stream: Tk100Stream, word: *mut u32) -> Tk100Status;
    pub fn tk100_launch_count(ctx: *const Tk100Ctx) -> u64;
    pub fn tk100_last_kernel(ctx: *mut Tk100Ctx) -> *const c_char;

    pub fn tk100_rms_norm(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16, weight: *const u16,
        output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_residual_rms_norm(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, residual_input: *const u16,
        branch: *const u16, weight: *const u16, residual_output: *mut u16,
        normalized_output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_residual_rms_norm_quantize(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, residual_input: *const u16,
        branch: *const u16, weight: *const u16, residual_output: *mut u16,
        normalized_output: *mut u16, activation_codes: *mut u8, activation_scales: *mut f32,
    ) -> Tk100Status;
    pub fn tk100_residual_rms_norm_quantize_nvfp4(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, residual_input: *const u16,
        branch: *const u16, weight: *const u16, residual_output: *mut u16,
        normalized_output: *mut u16, activation_codes: *mut u8, activation_scales: *mut f32,
        input_global_divisor: f32, nvfp4_codes: *mut u8, nvfp4_scales: *mut u8,
    ) -> Tk100Status;
    pub fn tk100_quantize_activation_e4m3(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, columns: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32,
    ) -> Tk100Status;

    pub fn tk100_fp8_qkv(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, out_rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_gdn_input(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, out_rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_projection(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, out_rows: c_int, columns: c_int,
        input: *const u16, activation_codes: *mut u8, activation_scales: *mut f32,
        weight_codes: *const u8, weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_swiglu(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_down(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_gdn_output(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, columns: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_register_plane(
        ctx: *mut Tk100Ctx, weight_codes: *const c_void, rows: u64, row_bytes: u64,
    ) -> Tk100Status;
    pub fn tk100_tensor_map_counts(ctx: *const Tk100Ctx, registered: *mut u64, transient: *mut u64);
    pub fn tk100_materialize_gather(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, planes: c_int, sources: *const *const c_void,
        bytes: *const u64, output: *mut c_void,
    ) -> Tk100Status;
    pub fn tk100_materialize_nvfp4_scales(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, planes: c_int, sources: *const *const u8,
        rows_per_plane: u64, groups_per_row: u64, output: *mut u8,
    ) -> Tk100Status;
    pub fn tk100_sample(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, vocab: c_int, logits: *const u16,
        options: *const Tk100SamplingOptions, rng_state: *mut u64, scratch: *mut u64,
        decisions: *mut Tk100SampleDecision, top_out: *mut u32,
    ) -> Tk100Status;
    pub fn tk100_sampler_initial_state(seed: u64) -> u64;
    pub fn tk100_sampler_scratch_bytes(rows: c_int, vocab: c_int) -> usize;
    pub fn tk100_gdn_prepare(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, batch: c_int, input: *const u16,
        control_weights: *const u16, a_log: *const u16, dt_bias: *const u16,
        projected: *const u16, convolution_weights: *const u16, state_rows: *const u32,
        history: *mut u16, log_decay: *mut f32, beta: *mut f32, convolved: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_gdn_recurrence(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, batch: c_int, qkv: *const u16,
        projected: *const u16, log_decay: *const f32, beta: *const f32, norm_weight: *const u16,
        state_rows: *const u32, state: *mut f32, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_fp8_lm_head(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, vocab_rows: c_int, vocab_offset: c_int,
        input: *const u16, activation_codes: *mut u8, activation_scales: *mut f32,
        weight_codes: *const u8, weight_scales: *const u16, output: *mut u16, logits_f32: *mut f32,
        argmax_scratch: *mut u64, pairs: *mut Tk100ArgmaxPair,
    ) -> Tk100Status;
    pub fn tk100_fp8_lm_head_sharded(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, vocab_rows: c_int, vocab_offset: c_int,
        input: *const u16, activation_codes: *mut u8, activation_scales: *mut f32,
        weight_codes: *const u8, weight_scales: *const u16, output: *mut u16, logits_f32: *mut f32,
        argmax_scratch: *mut u64, world: c_int, rank: c_int, peer_buffers: *const u64,
        merged_pairs: *mut Tk100ArgmaxPair,
    ) -> Tk100Status;
    pub fn tk100_argmax_merge(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, shards: c_int,
        gathered: *const Tk100ArgmaxPair, output: *mut Tk100ArgmaxPair,
    ) -> Tk100Status;
    pub fn tk100_argmax_exchange(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, world: c_int, rank: c_int,
        argmax_scratch: *mut u64, peer_buffers: *const u64, output: *mut Tk100ArgmaxPair,
    ) -> Tk100Status;

    pub fn tk100_nvfp4_quantize_activation(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, columns: c_int, input: *const u16,
        input_global_divisor: f32, activation_codes: *mut u8, activation_scales: *mut u8,
    ) -> Tk100Status;
    pub fn tk100_nvfp4_gate_up_swiglu(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
        weight_codes: *const u8, weight_scales: *const u8, weight_scale_divisor: f32,
        output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_peer_sum_bytes(capacity_values: usize, world: c_int) -> usize;
    pub fn tk100_peer_sum_bf16(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, values: usize, capacity_values: usize,
        world: c_int, rank: c_int, partial: *const f32, peer_buffers: *const u64, output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_nvfp4_gate_up_swiglu_quantize(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
        weight_codes: *const u8, weight_scales: *const u8, weight_scale_divisor: f32,
        output: *mut u16, output_global_divisor: f32, output_codes: *mut u8,
        output_scales: *mut u8,
    ) -> Tk100Status;
    pub fn tk100_nvfp4_down(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
        weight_codes: *const u8, weight_scales: *const u8, weight_scale_divisor: f32,
        output: *mut u16,
    ) -> Tk100Status;
    pub fn tk100_nvfp4_down_partial(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, rows: c_int, input: *const u16,
        activation_codes: *mut u8, activation_scales: *mut u8, input_global_divisor: f32,
        weight_codes: *const u8, weight_scales: *const u8, weight_scale_divisor: f32,
        partial_output: *mut f32,
    ) -> Tk100Status;
    pub fn tk100_f32_to_bf16(
        ctx: *mut Tk100Ctx, stream: Tk100Stream, count: usize, input: *const f32, output: *mut u16,
    ) -> Tk100Status;

    pub fn tk100_fp8_projection_static(
        stream: Tk100Stream, rows: c_int, out_rows: c_int, columns: c_int,
        activation_codes: *const u8, activation_scales: *const f32, weight_codes: *const u8,
        weight_scales: *const u16, output: *mut u16, message: *mut c_char,
        message_capacity: usize,
    ) -> Tk100Status;
    pub fn tk100_fp8_projection_static_status(stream: Tk100Stream, word: *mut u32) -> Tk100Status;
}
