"""Norms over the 32-bit residual stream (with the residual addition fused):
RMSNorm, and LayerNorm with weight and bias, which also reads a stream kept
in several copies.

Reference: rmsnorm (python/lyapunov_engine/ops.py:12-51) and rmsnorm_kernel
(csrc/kernels/fused_rmsnorm_swiglu.cu:15-113); the layer's norm weights there
are bare parameters of the decoder layer (python/lyapunov_engine/models/llama.py:130-134).
"""
from __future__ import annotations

from .. import ops
from .base import Norm, NormedAddend, ScaledAddend, TensorDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """``groups`` > 1: the row is cut into that many equal consecutive parts,
    each divided by its own sqrt(mean(part^2) + eps), before the weight.
    ``offset`` c: the stored weight lies around zero and the factor is c + w
    (made once at load, in 32 bits).

    It also reads a stream whose pending output enters normed
    (``NormedAddend``), and two such norms of the same stream run as one kernel
    (``apply_pair``: sub-layers that read the stream side by side)."""

    def __init__(self, hidden_size: int, eps: float, weight_name: str, groups: int = 1, offset: float = 0.0):
        self.hidden_size = int(hidden_size)
        self.groups = int(groups)
        self.offset = float(offset)
        if self.groups < 1 or self.hidden_size % self.groups:
            raise ValueError(f"a norm over {hidden_size} values cannot be cut into {groups} equal parts")
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.hidden_size,), role="vector",
                           init="taps" if self.offset else "ones_jitter")]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()
        self.runtime = runtime

    def apply(self, resid, delta=None, rows=None, workspace=None, key="normed", delta_scale=None):
        """``delta_scale`` (32-bit [hidden]): the delta enters the stream times it."""
        n = resid.shape[0] if rows is None else rows.shape[0]
        ws = workspace or self.runtime.workspace
        out = ws.get(key, (n, self.hidden_size), self.runtime.dtype)
        ops.rmsnorm(out, resid, delta, self.weight, self.eps, rows, groups=self.groups, delta_scale=delta_scale)
        return out

    def apply_stream(self, stream, read=None, rows=None, workspace=None, key="normed"):
        if isinstance(stream.update, ScaledAddend) and stream.copies == 1 and read is None:
            out = self.apply(stream.resid, stream.pending, rows=rows, workspace=workspace, key=key,
                             delta_scale=stream.update.weight if stream.pending is not None else None)
            if rows is None:
                stream.pending = stream.update = None
            return out
        if not isinstance(stream.update, NormedAddend):
            return super().apply_stream(stream, read, rows, workspace, key)
        return self.apply_pair(stream, None, rows=rows, workspace=workspace, keys=(key, None))[0]

    def apply_pair(self, stream, other: "RMSNorm | None", rows=None, workspace=None, keys=("normed", "normed_2")):
        """(this norm's output, ``other``'s) of the same stream, whose pending
        output enters first, plainly or normed, in one kernel.  Without
        ``rows`` the pending output is consumed."""
        if stream.copies != 1 or self.groups != 1 or (other is not None and (other.groups != 1 or other.eps != self.eps)):
            raise ValueError("norms that run as a pair read one copy of the stream, whole rows, with one eps")
        update = stream.update
        if update is not None and not isinstance(update, NormedAddend):
            raise ValueError(f"{type(self).__name__} cannot apply a pending {type(update).__name__}")
        n = stream.resid.shape[0] if rows is None else rows.shape[0]
        ws = workspace or self.runtime.workspace
        out1 = ws.get(keys[0], (n, self.hidden_size), self.runtime.dtype)
        out2 = ws.get(keys[1], (n, self.hidden_size), self.runtime.dtype) if other is not None else None
        ops.rmsnorm_pair(out1, out2, stream.resid, self.weight, other.weight if other is not None else None, self.eps,
                         addend=stream.pending, addend_weight=update.weight if update is not None else None,
                         addend_eps=update.eps if update is not None else 0.0, rows=rows)
        if rows is None:
            stream.pending = stream.update = None
        return out1, out2


@register_norm("layernorm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w + b with var the mean of the squared
    deviations, in 32 bits.  It reads a residual stream in one copy or in
    several (see ``apply_stream``): the pending update of the copies, the
    reading sub-layer's weighted sum of them and the norm are one kernel."""

    def __init__(self, hidden_size: int, eps: float, weight_name: str, bias_name: str):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight = self.bias = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.hidden_size,), role="vector", init="ones_jitter"),
                TensorDecl(self.bias_name, (self.hidden_size,), role="vector", init="zeros")]

    def bind(self, get, runtime):
        self.weight, self.bias = get(self.weight_name), get(self.bias_name)
        self.runtime = runtime

    def _out(self, n, workspace, key):
        ws = workspace or self.runtime.workspace
        return ws.get(key, (n, self.hidden_size), self.runtime.dtype)

    def apply(self, resid, delta=None, rows=None, workspace=None, key="normed"):
        out = self._out(resid.shape[0] if rows is None else rows.shape[0], workspace, key)
        ops.stream_norm(out, resid.view(resid.shape[0], 1, self.hidden_size), self.weight, self.bias, self.eps, delta=delta,
                        rows=rows)
        return out

    def apply_stream(self, stream, read=None, rows=None, workspace=None, key="normed"):
        T, W = stream.resid.shape[0], self.hidden_size
        copies = read.copies if read is not None else stream.copies
        init = None
        if stream.copies != copies:
            # the first sub-layer that keeps several copies: each starts as the one there is
            if stream.copies != 1 or stream.pending is not None or rows is not None:
                raise ValueError(f"a stream in {stream.copies} copies cannot be read as {copies}")
            init = stream.resid
            ws = workspace or self.runtime.workspace
            stream.resid = ws.get("stream_copies", (T, copies, W), init.dtype)
            stream.copies = copies
        out = self._out(T if rows is None else rows.shape[0], workspace, key)
        update = stream.update
        ops.stream_norm(out, stream.resid.view(T, copies, W), self.weight, self.bias, self.eps, delta=stream.pending,
                        mix=update.mix if update is not None else None, post=update.post if update is not None else None,
                        pre=read.pre if read is not None else None, init=init, rows=rows)
        if rows is None:
            stream.pending = stream.update = None
        return out
