"""Grouped-query attention over the paged cache, with per-head q/k RMSNorm.

qkv = x . Wqkv^T packed as [q | k | v] (tinyvllm/models/qwen3.py:230-240,
:273-280); q and k are normalised per head and rotated, k and v go to their
cache pages (:284-299; tinyvllm/kernels/kv_store.cu:26-90); every query attends
the keys of its request up to its own position, at most ``window`` of them
(tinyvllm/runtime/attention.py:34-55; tinyvllm/kernels/paged_decode.cu:85-466);
then the output projection (:303).  All sizes, the scale, the eps and the window
are parameters; the position encoding is a part of its own.
"""

from __future__ import annotations

import torch

from ..ops import attention as attention_ops
from ..ops import kernels, linear, linear_into_stream, linear_norm
from .base import BuildContext, KVNeed, ParamSpec, Part
from .registry import register_part


class GQAAttention(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, qk_norm_eps: float | None, window: int | None,
                 position=None, names: dict | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key-value heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"the attention kernels take head sizes in steps of 16 up to 256, not {head_dim}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.prefix = ctx.prefix
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        self.qkv_weight = self.o_weight = self.q_norm_weight = self.k_norm_weight = None

    # ------------------------------------------------------------ declaration
    def param_specs(self):
        q_rows, kv_rows = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = [
            ParamSpec.packed("qkv_weight", [(self.names["q"], q_rows), (self.names["k"], kv_rows),
                                            (self.names["v"], kv_rows)], self.hidden_size),
            ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, q_rows)),
        ]
        if self.qk_norm_eps is not None:
            specs += [
                ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
                ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
            ]
        return specs

    def children(self):
        return [self.position] if self.position is not None else []

    def streamed_weights(self):
        return [self.qkv_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        """Whether this mixer's prefill may run on the tcgen05 tile kernel; the step cuts its
        tile lists for that kernel only if every mixer of the model says so."""
        return kernels.attention_prefill_tc_supports(self.head_dim, self.num_heads, self.num_kv_heads,
                                                     page_size)

    def scratch_floats(self, rows: int, chunks: int) -> int:
        """float32 scratch the row kernel asks for when it spreads ``chunks`` key chunks of
        ``rows`` single tokens over the grid."""
        return kernels.attention_rows_scratch_floats(rows, self.num_heads, self.head_dim, chunks)

    # ---------------------------------------------------------------- running
    def forward(self, x, ctx, run: int):
        qkv = linear(x, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear(attended, self.o_weight)

    def forward_normed(self, hidden, residual, norm, ctx, run: int):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the output projection has added it to the stream itself."""
        qkv, residual = linear_norm(hidden, residual, norm, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear_into_stream(attended, self.o_weight, residual)


class WindowedAttention(Part):
    """Grouped-query attention with every size and step a parameter.

    Keys (``key_dim``) and values (``value_dim``) may differ in size.  ``qk_norm``: None, "unit"
    (q and k divided by their root mean square over the head, no weight) or "weight" (with
    tensors ``q_norm`` / ``k_norm``); ``position``: a position part whose ``inv_freq``, ``rot_dims``
    and ``pairing`` the preparing kernel applies to q and k, or None (positions then do not enter
    the scores).  ``window``: query i sees the keys j with 0 <= i - j < window, and with
    ``keep_first`` also the keys j < keep_first.  ``gate``: the concatenated heads are multiplied
    by sigmoid(W_g x) before the output projection.  ``value_mix``: "first" hands this layer's
    values on to the later layers of the step under ``value_mix_key``; "blend" replaces v by
    (1 - l) v + l v_first, with the scalar tensor ``vmix`` as l, before it is cached.

    ``hosted=True``: a block computes the input projections of all its parts as one product and
    the output projections as another; the mixer then owns no matrices, names its share
    (``input_rows``, ``output_cols``) and works between the two products (``between``)."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 key_dim: int, value_dim: int, scale: float, window: int | None = None,
                 keep_first: int = 0, qk_norm: str | None = None, qk_norm_eps: float = 0.0,
                 position=None, gate: bool = False, value_mix: str | None = None,
                 value_mix_key: str = "v_first", names: dict | None = None, hosted: bool = False) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key-value heads")
        if not 0 < key_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"the attention kernels take key and value sizes up to 256, not {key_dim} / {value_dim}")
        if qk_norm not in (None, "unit", "weight"):
            raise ValueError(f"qk_norm is None, 'unit' or 'weight', not {qk_norm!r}")
        if value_mix not in (None, "first", "blend"):
            raise ValueError(f"value_mix is None, 'first' or 'blend', not {value_mix!r}")
        if window is not None and window <= 0:
            raise ValueError("a window holds at least one key")
        if keep_first < 0:
            raise ValueError("keep_first must not be negative")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale = float(scale)
        self.window = window
        self.keep_first = keep_first if window is not None else 0
        self.qk_norm, self.qk_norm_eps = qk_norm, float(qk_norm_eps)
        self.gate = gate
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.hosted = hosted
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "vmix": "vmix", "q_norm": "q_norm",
             "k_norm": "k_norm", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        self.in_weight = self.o_weight = self.vmix = self.q_norm_weight = self.k_norm_weight = None

    # ------------------------------------------------------------ declaration
    @property
    def q_cols(self) -> int:
        return self.num_heads * self.key_dim

    @property
    def k_cols(self) -> int:
        return self.num_kv_heads * self.key_dim

    @property
    def v_cols(self) -> int:
        return self.num_kv_heads * self.value_dim

    @property
    def out_cols(self) -> int:
        return self.num_heads * self.value_dim

    def input_rows(self):
        """(checkpoint tensor, rows) of the input projections, in the order of their columns:
        q heads, k heads, v heads and, with a gate, the gate."""
        rows = [(self.names["q"], self.q_cols), (self.names["k"], self.k_cols), (self.names["v"], self.v_cols)]
        if self.gate:
            rows.append((self.names["g"], self.out_cols))
        return rows

    def output_cols(self):
        return (self.names["o"], self.out_cols)

    def param_specs(self):
        specs = []
        if not self.hosted:
            specs += [ParamSpec.packed("in_weight", self.input_rows(), self.hidden_size),
                      ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, self.out_cols))]
        if self.value_mix is not None:
            # every layer that takes part stores the scalar; the one that hands its values on ignores it
            specs.append(ParamSpec.scalar("vmix", self.names["vmix"]))
        if self.qk_norm == "weight":
            specs += [ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.key_dim,),
                                       role="vector", init="around_one"),
                      ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.key_dim,),
                                       role="vector", init="around_one")]
        return specs

    def children(self):
        return [self.position] if self.position is not None else []

    def streamed_weights(self):
        return [] if self.hosted else [self.in_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.key_dim, self.window, self.value_dim, self.keep_first)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        return False

    def scratch_floats(self, rows: int, chunks: int) -> int:
        """float32 scratch for ``rows`` single tokens whose keys span ``chunks`` chunks: what the row
        kernel or the tensor-core kernel for single tokens asks for, whichever is more."""
        span = chunks * kernels.attention_chunk_keys()
        return max(kernels.attention_rows_scratch_floats(rows, self.num_heads, self.value_dim, chunks),
                   kernels.attention_tiles_singles_floats(rows, self.num_heads, self.value_dim, self.window,
                                                          self.keep_first, span))

    # ---------------------------------------------------------------- running
    def between(self, projected, at: int, ctx, out, run: int) -> None:
        """From this mixer's columns of a projection (from ``at`` on) to the gated, concatenated
        heads in ``out``; writes the step's keys and values."""
        attention_ops.windowed_attention(ctx, self, projected, at, run, out)

    def forward(self, x, ctx, run: int):
        projected = linear(x, self.in_weight)
        attended = torch.empty((x.shape[0], self.out_cols), dtype=x.dtype, device=x.device)
        self.between(projected, 0, ctx, attended, run)
        return linear(attended, self.o_weight)


register_part("mixer", "gqa_attention", GQAAttention)
register_part("mixer", "windowed_attention", WindowedAttention)
