"""FP64 oracle of the gated-delta-net decode steps (numpy).

Test infrastructure only: imported by ``tests/`` and the smoke check, never by the shipped
package.  It restates the two FP64 formulas the reference qualifies its device code against:

* ``gdn_prepare``   -- qual/src/gdn_prepare.rs:333-431 (controls :333-373, convolution and the
  history shift :375-431);
* ``gdn_recurrence`` -- qual/src/gdn_recurrence.rs:274-335.

The reference's tests hold no numeric known answers for these operators: its gate is "device
within a tolerance of this formula on the generated fixture".  The restatement is therefore pinned
by (a) the reference's fixture generators, reproduced in ``tests/fixtures_ref.py``, and (b) a
scalar pure-Python re-evaluation of sampled elements in ``tests/test_oracle_gdn.py``.

BF16 planes travel as ``uint16`` bit patterns, controls and state as floating point arrays.
"""
from __future__ import annotations

import numpy as np

HEAD_DIM = 128
KEY_HEADS = 16
VALUE_HEADS = 48
QK_WIDTH = KEY_HEADS * HEAD_DIM
VALUE_WIDTH = VALUE_HEADS * HEAD_DIM
QKV_ROWS = 2 * QK_WIDTH + VALUE_WIDTH          # 10240
INPUT_ROWS = QKV_ROWS + VALUE_WIDTH            # 16384
CONTROL_ROWS = VALUE_HEADS                     # 48
HISTORY_TAPS = 3
RMS_EPSILON = 1.0e-6
DELTA_SCALE = 0.088_388_35


def _bf16(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def gdn_controls(input_bf16, control_weights_bf16, a_log_bf16, dt_bias_bf16):
    """(log_decay, beta), each ``[batch, 48]`` f64.  qual/src/gdn_prepare.rs:333-373."""
    x = _bf16(input_bf16)                      # [batch, hidden]
    w = _bf16(control_weights_bf16)            # [96, hidden]
    sums = x @ w.T                             # [batch, 96]
    control = sums[:, :CONTROL_ROWS] + _bf16(dt_bias_bf16)[None, :]
    log_decay = -np.exp(_bf16(a_log_bf16))[None, :] * np.log(1.0 + np.exp(control))
    beta = 1.0 / (1.0 + np.exp(-sums[:, CONTROL_ROWS:]))
    return log_decay, beta


def gdn_convolution(projected_bf16, convolution_weights_bf16, state_rows, history_bf16):
    """(convolved f64 ``[batch, 10240]``, history after the shift as uint16).

    ``history_bf16`` is ``[state rows, 10240, 3]``; tokens are applied in order, as the
    reference's loop does (qual/src/gdn_prepare.rs:375-431)."""
    projected = np.ascontiguousarray(projected_bf16, dtype=np.uint16)
    history = np.array(history_bf16, dtype=np.uint16, copy=True).reshape(-1, QKV_ROWS, HISTORY_TAPS)
    w = _bf16(convolution_weights_bf16).reshape(QKV_ROWS, 4)
    batch = projected.shape[0]
    out = np.zeros((batch, QKV_ROWS), dtype=np.float64)
    for token in range(batch):
        row = int(state_rows[token])
        current = projected[token, :QKV_ROWS]
        taps = np.concatenate([history[row], current[:, None]], axis=1)   # [10240, 4] bits
        total = (w * _bf16(taps)).sum(axis=1)
        out[token] = total / (1.0 + np.exp(-total))
        history[row] = taps[:, 1:]
    return out, history


def gdn_recurrence(qkv_bf16, projected_bf16, log_decay, beta, norm_weight_bf16, state_rows, state):
    """(state after the update f64 ``[rows, 48, 128, 128]``, output f64 ``[batch, 6144]``).

    qual/src/gdn_recurrence.rs:274-335."""
    qkv = _bf16(qkv_bf16)
    projected = _bf16(projected_bf16)
    norm_weight = _bf16(norm_weight_bf16)
    state = np.array(state, dtype=np.float64, copy=True).reshape(-1, VALUE_HEADS, HEAD_DIM, HEAD_DIM)
    log_decay = np.asarray(log_decay, dtype=np.float64).reshape(-1, VALUE_HEADS)
    beta = np.asarray(beta, dtype=np.float64).reshape(-1, VALUE_HEADS)
    batch = qkv.shape[0]
    output = np.zeros((batch, VALUE_WIDTH), dtype=np.float64)
    for token in range(batch):
        row = int(state_rows[token])
        q = qkv[token, :QK_WIDTH].reshape(KEY_HEADS, HEAD_DIM)
        k = qkv[token, QK_WIDTH:2 * QK_WIDTH].reshape(KEY_HEADS, HEAD_DIM)
        q = q / np.sqrt((q * q).sum(axis=1, keepdims=True) + RMS_EPSILON)
        k = k / np.sqrt((k * k).sum(axis=1, keepdims=True) + RMS_EPSILON)
        value = qkv[token, 2 * QK_WIDTH:].reshape(VALUE_HEADS, HEAD_DIM)
        gate = projected[token, QKV_ROWS:QKV_ROWS + VALUE_WIDTH].reshape(VALUE_HEADS, HEAD_DIM)
        for head in range(VALUE_HEADS):
            key_head = head // (VALUE_HEADS // KEY_HEADS)
            decay = np.exp(log_decay[token, head])
            s = state[row, head]                                  # [row, column]
            state_key = s @ k[key_head]                           # per state row
            update = beta[token, head] * (value[head] - decay * state_key)
            s = decay * s + update[:, None] * k[key_head][None, :]
            state[row, head] = s
            recurrent = (s @ q[key_head]) * DELTA_SCALE
            rms = np.sqrt((recurrent * recurrent).sum() / HEAD_DIM + RMS_EPSILON)
            silu = gate[head] / (1.0 + np.exp(-gate[head]))
            output[token, head * HEAD_DIM:(head + 1) * HEAD_DIM] = recurrent / rms * norm_weight * silu
    return state, output
