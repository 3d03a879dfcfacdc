"""Python mirror of the reference's prepared operators over the C ABI.

Names, argument order and error classes follow the reference
(``ResidualNormOp::launch_plain/launch_residual``, ``FullAttentionQkvOp::launch``,
``GdnInputProjectionOp::launch``, ``LmHeadOp::launch``).  Planes are torch CUDA tensors
(or raw integer device addresses); BF16 planes may be ``torch.bfloat16`` or ``uint16``/
``int16`` bit views.  Nothing here computes: every method is one C-ABI call.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib


class GpuError(RuntimeError):
    """Failure with the reference's stable category (``gpu.launch``, ``gpu.driver``, ...)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.code = _lib.STATUS_NAMES.get(status, f"gpu.unknown({status})")


def _ptr(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not t.is_cuda:
        raise GpuError(4, "[gpu.context] plane is not a CUDA tensor")
    if not t.is_contiguous():
        raise GpuError(5, "[gpu.launch] plane is not contiguous")
    return t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Context:
    """Owns one ``tk100_ctx`` (one per GPU / rank)."""

    def __init__(self, device: int = 0, hidden: int = 5120, intermediate: int = 17408,
                 rms_norm_epsilon: float = 1e-6, max_rows: int = 2048,
                 workspace_bytes: int = 0):
        self._lib = _lib.load()
        cfg = _lib.Config(_lib.ABI_VERSION, device, hidden, intermediate, rms_norm_epsilon,
                          max_rows, workspace_bytes)
        handle = C.c_void_p()
        status = self._lib.tk100_create(C.byref(cfg), C.byref(handle))
        if status != 0:
            raise GpuError(status, (self._lib.tk100_last_error(None) or b"").decode())
        self.handle = handle
        self.device = device
        self.hidden = hidden
        self.intermediate = intermediate

    def close(self):
        if getattr(self, "handle", None):
            self._lib.tk100_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status: int):
        if status != 0:
            raise GpuError(status, (self._lib.tk100_last_error(self.handle) or b"").decode())

    def device_status(self, stream=None) -> int:
        word = C.c_uint32(0)
        self.check(self._lib.tk100_device_status(self.handle, _stream(stream), C.byref(word)))
        return word.value

    def register_plane(self, weight_codes) -> None:
        """Encodes the TMA tensor map of a 2-D weight-code plane now (tk100_register_plane)."""
        rows, row_bytes = weight_codes.shape[0], weight_codes.shape[1] * weight_codes.element_size()
        self.check(self._lib.tk100_register_plane(self.handle, _ptr(weight_codes), rows, row_bytes))

    @property
    def tensor_map_counts(self):
        """(registered, lazily cached) tensor maps."""
        registered, transient = C.c_uint64(0), C.c_uint64(0)
        self._lib.tk100_tensor_map_counts(self.handle, C.byref(registered), C.byref(transient))
        return registered.value, transient.value

    @property
    def launch_count(self) -> int:
        return int(self._lib.tk100_launch_count(self.handle))

    @property
    def last_kernel(self) -> str:
        """Kernel instantiation of the last projection launch (``tk100_last_kernel``)."""
        return (self._lib.tk100_last_kernel(self.handle) or b"").decode()


class ResidualNormOp:
    """tuisko-kernels-sm120/src/residual_norm.rs:382-508."""

    def __init__(self, context: Context):
        self.ctx = context

    def launch_plain(self, stream, batch, input, weight, output):
        c = self.ctx
        c.check(c._lib.tk100_rms_norm(c.handle, _stream(stream), batch, _ptr(input), _ptr(weight),
                                      _ptr(output)))

    def launch_residual(self, stream, batch, residual_input, branch, weight, residual_output,
                        normalized_output):
        c = self.ctx
        c.check(c._lib.tk100_residual_rms_norm(c.handle, _stream(stream), batch,
                                               _ptr(residual_input), _ptr(branch), _ptr(weight),
                                               _ptr(residual_output), _ptr(normalized_output)))

    def launch_quantize(self, stream, batch, residual_input, branch, weight, residual_output,
                        normalized_output, activation_codes, activation_scales):
        """Fused producer: (residual add +) RMSNorm + per-token E4M3 quantisation, one kernel."""
        c = self.ctx
        c.check(c._lib.tk100_residual_rms_norm_quantize(
            c.handle, _stream(stream), batch, _ptr(residual_input), _ptr(branch), _ptr(weight),
            _ptr(residual_output), _ptr(normalized_output), _ptr(activation_codes),
            _ptr(activation_scales)))


    def launch_quantize_nvfp4(self, stream, batch, residual_input, branch, weight, residual_output,
                              normalized_output, activation_codes, activation_scales,
                              input_global_divisor, nvfp4_codes, nvfp4_scales):
        """Fused producer with both quantised forms: E4M3 (optional) and NVFP4, one kernel."""
        c = self.ctx
        c.check(c._lib.tk100_residual_rms_norm_quantize_nvfp4(
            c.handle, _stream(stream), batch, _ptr(residual_input), _ptr(branch), _ptr(weight),
            _ptr(residual_output), _ptr(normalized_output), _ptr(activation_codes),
            _ptr(activation_scales), input_global_divisor, _ptr(nvfp4_codes), _ptr(nvfp4_scales)))


class Fp8ProjectionOp:
    """Generic FP8 projection (any reduction length that is a multiple of 128)."""

    def __init__(self, context: Context):
        self.ctx = context

    def quantize(self, stream, rows, columns, input, activation_codes, activation_scales):
        c = self.ctx
        c.check(c._lib.tk100_quantize_activation_e4m3(c.handle, _stream(stream), rows, columns,
                                                      _ptr(input), _ptr(activation_codes),
                                                      _ptr(activation_scales)))

    def launch(self, stream, rows, out_rows, columns, input, activation_codes, activation_scales,
               weight_codes, weight_scales, output):
        c = self.ctx
        c.check(c._lib.tk100_fp8_projection(c.handle, _stream(stream), rows, out_rows, columns,
                                            _ptr(input), _ptr(activation_codes),
                                            _ptr(activation_scales), _ptr(weight_codes),
                                            _ptr(weight_scales), _ptr(output)))


class FullAttentionQkvOp:
    """tuisko-kernels-sm120/src/fp8/projection.rs:510-611; ``out_rows`` is a run-time value."""

    _entry = "tk100_fp8_qkv"

    def __init__(self, context: Context, out_rows: int):
        self.ctx = context
        self.out_rows = out_rows

    def launch(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
               weight_scales, output):
        c = self.ctx
        fn = getattr(c._lib, self._entry)
        c.check(fn(c.handle, _stream(stream), rows, self.out_rows, _ptr(input),
                   _ptr(activation_codes), _ptr(activation_scales), _ptr(weight_codes),
                   _ptr(weight_scales), _ptr(output)))


class GdnInputProjectionOp(FullAttentionQkvOp):
    """tuisko-kernels-sm120/src/fp8/projection.rs:613-702."""

    _entry = "tk100_fp8_gdn_input"


class Fp8SwiGluOp:
    """tuisko-kernels-sm120/src/fp8/swiglu.rs:366-376: dense-FP8 gate/up projection + SwiGLU;
    weights ``[2 * intermediate, hidden]`` with the gate rows first."""

    _entry = "tk100_fp8_swiglu"

    def __init__(self, context: Context):
        self.ctx = context

    def launch(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
               weight_scales, output):
        c = self.ctx
        fn = getattr(c._lib, self._entry)
        c.check(fn(c.handle, _stream(stream), rows, _ptr(input), _ptr(activation_codes),
                   _ptr(activation_scales), _ptr(weight_codes), _ptr(weight_scales), _ptr(output)))


class Fp8DownOp(Fp8SwiGluOp):
    """tuisko-kernels-sm120/src/fp8/down.rs:197-207: planes ``[rows, intermediate]`` in,
    ``[rows, hidden]`` out."""

    _entry = "tk100_fp8_down"


class GdnOutputProjectionOp:
    """tuisko-kernels-sm120/src/fp8/gdn_output.rs:178; ``columns`` = the GDN value width."""

    def __init__(self, context: Context, columns: int):
        self.ctx = context
        self.columns = columns

    def launch(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
               weight_scales, output):
        c = self.ctx
        c.check(c._lib.tk100_fp8_gdn_output(c.handle, _stream(stream), rows, self.columns, _ptr(input),
                                            _ptr(activation_codes), _ptr(activation_scales),
                                            _ptr(weight_codes), _ptr(weight_scales), _ptr(output)))


class Materializer:
    """Device counterpart of tuisko-model/src/materialize.rs: checkpoint planes, uploaded as stored,
    become the run-time planes without a host pass over their bytes."""

    def __init__(self, context: Context):
        self.ctx = context

    def gather(self, stream, planes, output=None):
        """``gather_source_planes`` (:295-314): the planes (1-D uint8 CUDA tensors) concatenated."""
        total = sum(p.numel() * p.element_size() for p in planes)
        if output is None:
            output = torch.empty(total, dtype=torch.uint8, device="cuda")
        c = self.ctx
        pointers = (C.c_void_p * len(planes))(*[_ptr(p) for p in planes])
        sizes = (C.c_uint64 * len(planes))(*[p.numel() * p.element_size() for p in planes])
        c.check(c._lib.tk100_materialize_gather(c.handle, _stream(stream), len(planes), pointers, sizes,
                                                _ptr(output)))
        return output

    def full_attention_qkv(self, stream, query_gate, key, value):
        """``FullAttentionQkvBindings::materialize`` (:33-103): each argument is a
        ``(weight_e4m3 [rows, columns] uint8, scale_bf16 [rows, 1])`` pair; returns the fused
        ``(weight, scale)`` planes in query/gate, key, value row order."""
        (qw, qs), (kw, ks), (vw, vs) = query_gate, key, value
        shapes_ok = (kw.shape[0] == vw.shape[0] and qw.shape[1] == kw.shape[1] == vw.shape[1]
                     and tuple(qs.shape) == (qw.shape[0], 1) and tuple(ks.shape) == (kw.shape[0], 1)
                     and tuple(vs.shape) == (vw.shape[0], 1))
        if not shapes_ok:
            raise GpuError(5, "[checkpoint.source_binding] full-attention QKV source planes have "
                              "incompatible shapes")
        rows = qw.shape[0] + kw.shape[0] + vw.shape[0]
        weight = self.gather(stream, [qw.reshape(-1), kw.reshape(-1), vw.reshape(-1)])
        scale = self.gather(stream, [t.reshape(-1).view(torch.uint8) for t in (qs, ks, vs)])
        return weight.view(rows, qw.shape[1]), scale.view(torch.int16).view(rows, 1)

    def nvfp4_scales(self, stream, planes, output=None):
        """``swizzle_scale_planes`` (:353-408): 1 or 2 row-major ``[rows, groups]`` uint8 planes ->
        one plane in 128 x 4 tiles.  Raises on a negative or NaN scale code like
        ``validate_nvfp4_scales`` (reads the device status word, so it synchronises)."""
        rows, groups = planes[0].shape
        if any(tuple(p.shape) != (rows, groups) for p in planes):
            raise GpuError(5, "[checkpoint.source_binding] NVFP4 source scale plane length does not "
                              "match its shape")
        if output is None:
            output = torch.empty(len(planes) * rows * groups, dtype=torch.uint8, device="cuda")
        c = self.ctx
        pointers = (C.c_void_p * len(planes))(*[_ptr(p) for p in planes])
        c.check(c._lib.tk100_materialize_nvfp4_scales(c.handle, _stream(stream), len(planes), pointers,
                                                      rows, groups, _ptr(output)))
        if c.device_status(stream) & _lib.DEVICE_BAD_ARGUMENT:
            raise GpuError(5, "[checkpoint.source_binding] NVFP4 scale plane contains a negative or "
                              "NaN E4M3FN code")
        return output


class SamplingOptions:
    """tuisko-engine/src/sampling.rs:11-45: per-request controls; ``greedy()`` and the defaults of
    the checkpoint's generation contract (temperature 1, top-p 0.95, top-k 20)."""

    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, seed=0):
        self.temperature, self.top_p, self.top_k, self.seed = temperature, top_p, top_k, seed

    @classmethod
    def greedy(cls):
        return cls(temperature=0.0, top_p=1.0, top_k=1, seed=0)


class Sampler:
    """Device counterpart of the reference's ``Sampler`` (tuisko-engine/src/sampling.rs:56-101) for a
    decode batch: one entry of ``options`` / ``stop_ids`` per request.  The generator states and the
    scratch live in device memory owned by this object; ``sample`` leaves the decisions
    ``[rows, 2]`` (token id, stopped) in ``self.decisions`` without a host round trip."""

    MAX_TOP_K = 32

    def __init__(self, context: Context, vocab: int, options, stop_ids):
        import torch

        self.ctx, self.vocab = context, vocab
        self.rows = len(options)
        lib = context._lib
        self._options = (_lib.SamplingOptions * self.rows)()
        for i, (o, stops) in enumerate(zip(options, stop_ids)):
            self._options[i].temperature = o.temperature
            self._options[i].top_p = o.top_p
            self._options[i].top_k = o.top_k
            self._options[i].stop_ids[0], self._options[i].stop_ids[1] = stops
        states = [lib.tk100_sampler_initial_state(o.seed) for o in options]
        self.rng_state = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in states],
                                      dtype=torch.int64, device="cuda")
        nbytes = lib.tk100_sampler_scratch_bytes(self.rows, vocab)
        self.scratch = torch.zeros((nbytes + 7) // 8, dtype=torch.int64, device="cuda")
        self.decisions = torch.zeros((self.rows, 2), dtype=torch.int32, device="cuda")
        self.top = torch.zeros((self.rows, self.MAX_TOP_K, 2), dtype=torch.int32, device="cuda")

    def sample(self, stream, logits, want_top: bool = False):
        c = self.ctx
        c.check(c._lib.tk100_sample(c.handle, _stream(stream), self.rows, self.vocab, _ptr(logits),
                                    self._options, _ptr(self.rng_state), _ptr(self.scratch),
                                    _ptr(self.decisions), _ptr(self.top) if want_top else None))


class GdnPrepareOp:
    """tuisko-kernels-sm120/src/gdn/prepare.rs:226-290: control mat-vecs and the width-4 causal
    convolution (with its in-place history shift) of a decode batch of 1..=8 tokens."""

    def __init__(self, context: Context):
        self.ctx = context

    def launch(self, stream, batch, input, control_weights, a_log, dt_bias, projected,
               convolution_weights, state_rows, history, log_decay, beta, convolved):
        c = self.ctx
        c.check(c._lib.tk100_gdn_prepare(
            c.handle, _stream(stream), batch, _ptr(input), _ptr(control_weights), _ptr(a_log),
            _ptr(dt_bias), _ptr(projected), _ptr(convolution_weights), _ptr(state_rows),
            _ptr(history), _ptr(log_decay), _ptr(beta), _ptr(convolved)))


class GdnRecurrenceOp:
    """tuisko-kernels-sm120/src/gdn/recurrence.rs:184-236: gated delta rule on the FP32 state
    (in place) and the gated RMSNorm of its outputs."""

    def __init__(self, context: Context):
        self.ctx = context

    def launch(self, stream, batch, qkv, projected, log_decay, beta, norm_weight, state_rows,
               state, output):
        c = self.ctx
        c.check(c._lib.tk100_gdn_recurrence(
            c.handle, _stream(stream), batch, _ptr(qkv), _ptr(projected), _ptr(log_decay),
            _ptr(beta), _ptr(norm_weight), _ptr(state_rows), _ptr(state), _ptr(output)))


class LmHeadOp:
    """tuisko-kernels-sm120/src/fp8/projection.rs:704-793 plus the fused greedy argmax.

    ``vocab_rows``/``vocab_offset`` describe this rank's shard of the vocabulary."""

    def __init__(self, context: Context, vocab_rows: int, vocab_offset: int = 0):
        self.ctx = context
        self.vocab_rows = vocab_rows
        self.vocab_offset = vocab_offset

    def launch(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
               weight_scales, output, logits_f32=None, argmax_scratch=None, pairs=None):
        c = self.ctx
        c.check(c._lib.tk100_fp8_lm_head(c.handle, _stream(stream), rows, self.vocab_rows,
                                         self.vocab_offset, _ptr(input), _ptr(activation_codes),
                                         _ptr(activation_scales), _ptr(weight_codes),
                                         _ptr(weight_scales), _ptr(output), _ptr(logits_f32),
                                         _ptr(argmax_scratch), _ptr(pairs)))

    def launch_sharded(self, stream, rows, input, activation_codes, activation_scales, weight_codes,
                       weight_scales, output, logits_f32, argmax_scratch, world, rank, peer_buffers,
                       merged_pairs):
        """Projection, per-shard argmax, peer exchange and merge in ONE launch
        (``tk100_fp8_lm_head_sharded``); ``peer_buffers`` may be None when ``world == 1``."""
        c = self.ctx
        arr = (C.c_uint64 * world)(*[int(b) for b in peer_buffers]) if peer_buffers else None
        c.check(c._lib.tk100_fp8_lm_head_sharded(
            c.handle, _stream(stream), rows, self.vocab_rows, self.vocab_offset, _ptr(input),
            _ptr(activation_codes), _ptr(activation_scales), _ptr(weight_codes), _ptr(weight_scales),
            _ptr(output), _ptr(logits_f32), _ptr(argmax_scratch), world, rank, arr,
            _ptr(merged_pairs)))

    def exchange(self, stream, rows, world, rank, argmax_scratch, peer_buffers, output_pairs):
        """Peer-store exchange + merge of the per-shard maxima (after ``launch`` with
        ``pairs=None``); ``peer_buffers`` lists every rank's exchange-buffer address."""
        c = self.ctx
        arr = (C.c_uint64 * world)(*[int(b) for b in peer_buffers])
        c.check(c._lib.tk100_argmax_exchange(c.handle, _stream(stream), rows, world, rank,
                                             _ptr(argmax_scratch), arr, _ptr(output_pairs)))

    def merge(self, stream, rows, shards, gathered_pairs, output_pairs):
        c = self.ctx
        c.check(c._lib.tk100_argmax_merge(c.handle, _stream(stream), rows, shards,
                                          _ptr(gathered_pairs), _ptr(output_pairs)))


def nvfp4_scale_plane_bytes(rows: int, columns: int) -> int:
    """Bytes of a swizzled NVFP4 scale plane: rows padded to 128, one byte per 16 columns."""
    return ((rows + 127) // 128) * 128 * (columns // 16)


class _Nvfp4Op:
    _entry = ""

    def __init__(self, context: Context):
        self.ctx = context

    def quantize(self, stream, rows, columns, input, input_global_divisor, activation_codes,
                 activation_scales):
        """NVFP4 activation quantiser (this library's own definition; see the header)."""
        c = self.ctx
        c.check(c._lib.tk100_nvfp4_quantize_activation(
            c.handle, _stream(stream), rows, columns, _ptr(input), input_global_divisor,
            _ptr(activation_codes), _ptr(activation_scales)))

    def launch(self, stream, batch, input, weight_codes, weight_scales, weight_scale_divisor,
               output, *, activation_codes, activation_scales, input_global_divisor):
        """The reference's argument order, followed by the W4A4 additions as keywords."""
        c = self.ctx
        fn = getattr(c._lib, self._entry)
        c.check(fn(c.handle, _stream(stream), batch, _ptr(input), _ptr(activation_codes),
                   _ptr(activation_scales), input_global_divisor, _ptr(weight_codes),
                   _ptr(weight_scales), weight_scale_divisor, _ptr(output)))


class Nvfp4SwiGluOp(_Nvfp4Op):
    """tuisko-kernels-sm89/src/nvfp4/swiglu.rs:470-571 (gate/up projection + SiLU * up)."""

    _entry = "tk100_nvfp4_gate_up_swiglu"

    def launch_quantize(self, stream, batch, input, weight_codes, weight_scales,
                        weight_scale_divisor, output, *, activation_codes, activation_scales,
                        input_global_divisor, output_global_divisor, output_codes, output_scales):
        """The same projection, also leaving the NVFP4 codes and block scales of its output for
        ``Nvfp4DownOp.launch(input=None, ...)`` (in the projection's epilogue up to 32 rows)."""
        c = self.ctx
        c.check(c._lib.tk100_nvfp4_gate_up_swiglu_quantize(
            c.handle, _stream(stream), batch, _ptr(input), _ptr(activation_codes),
            _ptr(activation_scales), input_global_divisor, _ptr(weight_codes),
            _ptr(weight_scales), weight_scale_divisor, _ptr(output), output_global_divisor,
            _ptr(output_codes), _ptr(output_scales)))


class Nvfp4DownOp(_Nvfp4Op):
    """tuisko-kernels-sm89/src/nvfp4/down.rs:455-556."""

    _entry = "tk100_nvfp4_down"

    def launch_partial(self, stream, batch, input, weight_codes, weight_scales,
                       weight_scale_divisor, partial_output, *, activation_codes,
                       activation_scales, input_global_divisor):
        """Row-parallel shard: unrounded fp32 partial sums for a later all-reduce."""
        c = self.ctx
        c.check(c._lib.tk100_nvfp4_down_partial(
            c.handle, _stream(stream), batch, _ptr(input), _ptr(activation_codes),
            _ptr(activation_scales), input_global_divisor, _ptr(weight_codes),
            _ptr(weight_scales), weight_scale_divisor, _ptr(partial_output)))


def f32_to_bf16(context: Context, stream, count, input, output):
    """fp32 -> BF16 (nearest even) of `count` values, e.g. after the tensor-parallel all-reduce."""
    context.check(context._lib.tk100_f32_to_bf16(context.handle, _stream(stream), count,
                                                 _ptr(input), _ptr(output)))


def peer_sum_bytes(capacity_values: int, world: int) -> int:
    """Size of one rank's exchange buffer for :func:`peer_sum_bf16` (tk100_peer_sum_bytes)."""
    return int(_lib.load().tk100_peer_sum_bytes(capacity_values, world))


def peer_sum_bf16(context: Context, stream, values, capacity_values, world, rank, partial,
                  peer_buffers, output):
    """BF16 sum over ranks of the fp32 ``partial`` (``values`` numbers, a multiple of 8) through
    the ranks' peer-mapped exchange buffers (``peer_buffers[i]`` = rank i's buffer address in this
    process, each ``peer_sum_bytes(capacity_values, world)`` bytes, zeroed once).  Every rank
    calls it; all ranks get identical bits."""
    arr = (C.c_uint64 * world)(*[int(b) for b in peer_buffers])
    context.check(context._lib.tk100_peer_sum_bf16(context.handle, _stream(stream), values,
                                                   capacity_values, world, rank, _ptr(partial), arr,
                                                   _ptr(output)))


def exchange_bytes(rows: int, world: int) -> int:
    """Size of one rank's peer exchange buffer (TK100_EXCHANGE_BYTES)."""
    return 2 * world * rows * 16


STATIC_MAX_ROWS = 256
STATIC_SCRATCH_BYTES = (8 << 20) + (16 << 10)


def fp8_projection_static(stream, rows, out_rows, columns, activation_codes, activation_scales,
                          weight_codes, weight_scales, output):
    """FP8 projection without a context, for hosts that may not allocate device memory (an
    engine with a fixed arena and a no-allocation gate, or guest code in a process whose
    allocator it does not own).  The split-K scratch is a fixed ``STATIC_SCRATCH_BYTES`` array
    inside the library that every GPU loading it keeps until exit; ``rows`` is limited to
    ``STATIC_MAX_ROWS`` and larger scratch needs are refused with ``gpu.arena``.  The first call
    on a device does the one-time set-up and should come before any stream capture; calls
    share the array, so calls that could overlap on the GPU must be serialised."""
    lib = _lib.load()
    message = C.create_string_buffer(320)
    status = lib.tk100_fp8_projection_static(_stream(stream), rows, out_rows, columns,
                                             _ptr(activation_codes), _ptr(activation_scales),
                                             _ptr(weight_codes), _ptr(weight_scales), _ptr(output),
                                             message, len(message))
    if status != 0:
        raise GpuError(status, message.value.decode())


def fp8_projection_static_status(stream=None) -> int:
    """Reads and clears the fault word of the static scratch on the current device (the
    ``TK100_DEVICE_*`` bits that :meth:`Context.device_status` reports for the context route)."""
    lib = _lib.load()
    word = C.c_uint32(0)
    status = lib.tk100_fp8_projection_static_status(_stream(stream), C.byref(word))
    if status != 0:
        raise GpuError(status, "[gpu.driver] reading the static scratch's fault word failed")
    return word.value
