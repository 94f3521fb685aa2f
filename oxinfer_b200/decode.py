"""Host mirror of the reference's ``gpu::decode`` module (``src/gpu_decode.rs``): a model describes one
token's forward pass as ops over activation buffers (``Graph``), the backend turns it into a plan
(``Backend.decode_plan``) and ``DecodePlan.step`` runs a whole token in one submission.

Only the op set of a dense Llama / Qwen3 layer is taken (Norm, Linear, QkRope, Attend, Glu); a graph
with anything else is declined, as ``decode_plan`` returns ``None`` in the reference and the model
decodes on the CPU. ``llama_graph`` builds the same op list as the Llama branch of
``QwenModel::gpu_graph_mode`` (``src/qwen.rs:1177-1528``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import MODE_ADD, MODE_SILU_PAIR, MODE_STORE, OP_ATTEND, OP_EXCHANGE, OP_GLU, OP_LINEAR, OP_NORM, OP_QK_ROPE, PLAN_HANDLE_BYTES


@dataclass(frozen=True)
class View:
    """A position inside an activation buffer, in floats (``src/gpu_decode.rs:21-35``)."""

    buf: int
    off: int = 0

    def at(self, off: int) -> "View":
        return View(self.buf, self.off + off)

    def c(self) -> _lib.View:
        return _lib.View(self.buf, self.off)


@dataclass
class Graph:
    """``Graph`` of ``src/gpu_decode.rs:378-416`` restricted to the fields the dense path uses."""

    bufs: list = field(default_factory=list)
    ops: list = field(default_factory=list)
    input: View = View(0)
    n_input: int = 0
    hidden: View = View(0)
    n_hidden: int = 0
    logits: tuple | None = None          # (View, n)
    kv: list = field(default_factory=list)           # (n_kv, hd) per cache
    rope_halves: list = field(default_factory=list)
    _keep: list = field(default_factory=list)        # host arrays the op structs point into

    def buf(self, n: int) -> View:
        self.bufs.append(int(n))
        return View(len(self.bufs) - 1, 0)

    # -- op constructors (Op::norm etc.) -----------------------------------------------------------
    def norm(self, x: View, out: View, w: np.ndarray | None, n: int, eps: float, rows: int = 1, pre: float = 1.0, add: bool = False,
             x_stride: int | None = None, out_stride: int | None = None) -> None:
        o = _lib.Op(kind=OP_NORM, x=x.c(), y=out.c(), n=n, rows=rows, x_stride=x_stride or n, out_stride=out_stride or n, add=int(add), pre=pre,
                    eps=eps)
        if w is not None:
            w = np.ascontiguousarray(w, dtype=np.float32)
            assert w.shape == (n,)
            self._keep.append(w)
            o.p0 = w.ctypes.data
        self.ops.append(o)

    def linear(self, dev, x: View, y: View, mode: int = MODE_STORE, dev2=None, gate: View | None = None) -> None:
        o = _lib.Op(kind=OP_LINEAR, x=x.c(), y=y.c(), w=dev.handle, w2=dev2.handle if dev2 is not None else 0, mode=mode, n_out=dev.n_out,
                    n_in=dev.n_in)
        if gate is not None:
            o.z = gate.c()
        self.ops.append(o)

    def qk_rope(self, qkv: View, q_out: View, kv: int, nh: int, nkv: int, hd: int, half_rot: int, k_off: int, v_off: int, interleaved: bool,
                eps: float, q_stride: int | None = None, q_norm: np.ndarray | None = None, k_norm: np.ndarray | None = None, rope: int = 0,
                v_norm: bool = False, v_from_k: bool = False) -> None:
        o = _lib.Op(kind=OP_QK_ROPE, x=qkv.c(), y=q_out.c(), kv=kv, nh=nh, nkv=nkv, hd=hd, half_rot=half_rot, q_stride=q_stride or hd,
                    k_off=k_off, v_off=v_off, interleaved=int(interleaved), rope=rope, v_norm=int(v_norm), v_from_k=int(v_from_k), eps=eps)
        for name, w in (("p0", q_norm), ("p1", k_norm)):
            if w is not None:
                w = np.ascontiguousarray(w, dtype=np.float32)
                assert w.shape == (hd,)
                self._keep.append(w)
                setattr(o, name, w.ctypes.data)
        self.ops.append(o)

    def attend(self, q: View, out: View, kv: int, nh: int, nkv: int, hd: int, scale: float, window: int | None = None) -> None:
        self.ops.append(_lib.Op(kind=OP_ATTEND, x=q.c(), y=out.c(), kv=kv, nh=nh, nkv=nkv, hd=hd, scale=scale, window=window or 0))

    def glu(self, g: View, u: View, out: View, n: int, gelu: bool = False) -> None:
        self.ops.append(_lib.Op(kind=OP_GLU, x=g.c(), z=u.c(), y=out.c(), n=n, gelu=int(gelu)))

    def exchange(self, x: View, n: int) -> None:
        """Tensor-parallel plans (no counterpart in the reference): every rank wrote its equal contiguous part of the
        ``n`` values at ``x``; afterwards every rank holds all of them."""
        self.ops.append(_lib.Op(kind=OP_EXCHANGE, x=x.c(), n=n))


class DecodePlan:
    """``DecodePlan`` (``src/gpu_decode.rs:538-587``) over the plan's own device KV caches."""

    def __init__(self, be, handle: int, graph: Graph, max_len: int):
        self._be, self.handle, self.graph, self.max_len = be, handle, graph, max_len
        self.cs_stride = 2 * sum(graph.rope_halves)

    def close(self) -> None:
        if self.handle:
            self._be._L.b2_plan_free(self._be._ctx, self.handle)
            self.handle = 0

    def launches_per_step(self) -> int:
        n = C.c_uint64()
        self._be._check(self._be._L.b2_plan_launches(self._be._ctx, self.handle, C.byref(n)))
        return n.value

    # -- tensor-parallel plans: one process per GPU, the same graph over each rank's weight shards -------------------
    def export_handle(self) -> bytes:
        """What the other ranks need to reach this plan's activation memory (pass it by any host-side means)."""
        buf = C.create_string_buffer(PLAN_HANDLE_BYTES)
        self._be._check(self._be._L.b2_plan_export(self._be._ctx, self.handle, buf))
        return buf.raw

    def attach_peers(self, rank: int, world: int, handles: list) -> None:
        """``handles``: every rank's ``export_handle()`` in rank order. Steps are collective from here on."""
        assert len(handles) == world and all(len(h) == PLAN_HANDLE_BYTES for h in handles)
        blob = b"".join(handles)
        self._be._check(self._be._L.b2_plan_attach_peers(self._be._ctx, self.handle, rank, world, blob))

    def step(self, pos: int, x: np.ndarray, rope_cs: np.ndarray, want_logits: bool = True):
        """One token: returns (hidden, logits or None); raises on error (there is no CPU path here)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        cs = np.ascontiguousarray(rope_cs, dtype=np.float32)
        assert x.size == self.graph.n_input and cs.size == self.cs_stride
        hidden = np.empty(self.graph.n_hidden, dtype=np.float32)
        logits = np.empty(self.graph.logits[1], dtype=np.float32) if want_logits and self.graph.logits else None
        self._be._check(self._be._L.b2_plan_step(self._be._ctx, self.handle, pos, x.ctypes.data, cs.ctypes.data, hidden.ctypes.data,
                                                 logits.ctypes.data if logits is not None else None))
        return hidden, logits

    def tokens(self) -> int:
        """``DecodePlan::tokens`` (``src/gpu_decode.rs:575-577``): the most tokens of a step."""
        n = C.c_size_t()
        self._be._check(self._be._L.b2_plan_tokens(self._be._ctx, self.handle, C.byref(n)))
        return n.value

    def step_multi(self, pos: int, x: np.ndarray, rope_cs: np.ndarray, want_logits: bool = True, hidden_out: np.ndarray | None = None):
        """``t`` tokens at positions ``pos .. pos + t - 1`` (``Step::t``, ``src/gpu_decode.rs:538-570``): ``x`` is ``[t][n_input]``,
        ``rope_cs`` holds, for each RoPE table in turn, ``t`` rows of cos then sin. Returns (hidden ``[t][n_hidden]``, logits
        ``[t][n_logits]`` or None); every row equals the result of a one-token step, bit for bit (a prefill plan's: up to
        rounding). ``hidden_out``: a caller's ``[t][n_hidden]`` f32 array to fill (page-locked memory makes the copies faster)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        t = x.shape[0]
        cs = np.ascontiguousarray(rope_cs, dtype=np.float32)
        assert x.ndim == 2 and x.shape[1] == self.graph.n_input and cs.size == t * self.cs_stride
        hidden = np.empty((t, self.graph.n_hidden), dtype=np.float32) if hidden_out is None else hidden_out
        assert hidden.dtype == np.float32 and hidden.flags["C_CONTIGUOUS"] and hidden.shape == (t, self.graph.n_hidden)
        logits = np.empty((t, self.graph.logits[1]), dtype=np.float32) if want_logits and self.graph.logits else None
        self._be._check(self._be._L.b2_plan_step_multi(self._be._ctx, self.handle, pos, t, x.ctypes.data, cs.ctypes.data, hidden.ctypes.data,
                                                       logits.ctypes.data if logits is not None else None))
        return hidden, logits

    def last_step_ms(self) -> float:
        """Device milliseconds of the kernels of the last prefill step (without the host copies)."""
        ms = C.c_float()
        self._be._check(self._be._L.b2_plan_last_step_ms(self._be._ctx, self.handle, C.byref(ms)))
        return ms.value

    def kv_write(self, kv: int, pos0: int, k: np.ndarray, v: np.ndarray) -> None:
        """Rows ``[n][n_kv][hd]`` f32 in the host cache's order into positions ``pos0 ..``."""
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        nkv, hd = self.graph.kv[kv]
        n = k.size // (nkv * hd)
        assert k.size == n * nkv * hd and v.size == k.size
        self._be._check(self._be._L.b2_plan_kv_write(self._be._ctx, self.handle, kv, pos0, n, k.ctypes.data, v.ctypes.data))

    def kv_read(self, kv: int, pos0: int, n: int):
        nkv, hd = self.graph.kv[kv]
        k = np.empty((n, nkv, hd), dtype=np.float32)
        v = np.empty((n, nkv, hd), dtype=np.float32)
        self._be._check(self._be._L.b2_plan_kv_read(self._be._ctx, self.handle, kv, pos0, n, k.ctypes.data, v.ctypes.data))
        return k, v

    def generate(self, embed, first_token: int, pos0: int, n_tokens: int, rope_cs_table: np.ndarray):
        """Greedy tokens without the host in the loop: returns (tokens int32 [n_tokens], device milliseconds)."""
        cs = np.ascontiguousarray(rope_cs_table, dtype=np.float32)
        assert cs.size == n_tokens * self.cs_stride
        out = np.empty(n_tokens, dtype=np.int32)
        ms = C.c_float()
        self._be._check(self._be._L.b2_plan_generate(self._be._ctx, self.handle, embed.handle, first_token, pos0, n_tokens, cs.ctypes.data,
                                                     out.ctypes.data, C.byref(ms)))
        return out, ms.value


def decode_plan(be, g: Graph, max_len: int, kv_f16: bool = False, tokens: int = 1, prefill: bool = False) -> DecodePlan | None:
    """``Backend::decode_plan`` (``src/gpu.rs:262-289``): a plan, or ``None`` when the graph is declined. ``tokens`` > 1:
    ``Backend::decode_plan_multi`` (``src/gpu.rs:273-276``), steps of up to that many tokens."""
    bufs = (C.c_uint64 * len(g.bufs))(*g.bufs)
    ops = (_lib.Op * len(g.ops))(*g.ops)
    nkv = (C.c_uint32 * max(1, len(g.kv)))(*[k[0] for k in g.kv])
    hd = (C.c_uint32 * max(1, len(g.kv)))(*[k[1] for k in g.kv])
    halves = (C.c_uint32 * max(1, len(g.rope_halves)))(*g.rope_halves)
    lv, ln = g.logits if g.logits else (View(0), 0)
    desc = _lib.GraphDesc(bufs=bufs, n_bufs=len(g.bufs), ops=ops, n_ops=len(g.ops), input=g.input.c(), n_input=g.n_input, hidden=g.hidden.c(),
                          n_hidden=g.n_hidden, logits=lv.c(), n_logits=ln, kv_nkv=nkv, kv_hd=hd, n_kv=len(g.kv), rope_halves=halves,
                          n_rope=len(g.rope_halves), max_len=max_len, kv_f16=int(kv_f16))
    h = C.c_uint64()
    if prefill:
        rc = be._L.b2_decode_plan_prefill(be._ctx, C.byref(desc), tokens, C.byref(h))
    elif tokens == 1:
        rc = be._L.b2_decode_plan(be._ctx, C.byref(desc), C.byref(h))
    else:
        rc = be._L.b2_decode_plan_multi(be._ctx, C.byref(desc), tokens, C.byref(h))
    if not be._check(rc):
        return None
    return DecodePlan(be, h.value, g, max_len)


def decode_plan_multi(be, g: Graph, max_len: int, tokens: int, kv_f16: bool = False) -> DecodePlan | None:
    """``Backend::decode_plan_multi`` (``src/gpu.rs:273-276``); also what ``decode_plan_multi_fast`` gives (the exact plan)."""
    return decode_plan(be, g, max_len, kv_f16=kv_f16, tokens=tokens)


def decode_plan_prefill(be, g: Graph, max_len: int, tokens: int, kv_f16: bool = False) -> DecodePlan | None:
    """``Backend::decode_plan_prefill`` (``src/gpu.rs:283-289``): steps of up to ``tokens`` tokens on batched kernels; the graph
    has no head. Steps go through ``DecodePlan.step_multi``."""
    return decode_plan(be, g, max_len, kv_f16=kv_f16, tokens=tokens, prefill=True)


# ---- RoPE tables (src/kernels.rs:2277-2306) ---------------------------------------------------------
def rope_inv_freq(dim: int, theta: float, proportion: float = 1.0) -> np.ndarray:
    half, rot = dim // 2, int(proportion * dim) // 2
    out = np.zeros(half, dtype=np.float32)
    for i in range(min(rot, half)):
        out[i] = np.float32(1.0 / theta ** ((2 * i) / dim))
    return out


def rope_table(pos: int, inv_freq: np.ndarray) -> np.ndarray:
    """cos[half] then sin[half] of one position, the angle an f32 product as in the reference."""
    a = np.float32(pos) * inv_freq.astype(np.float32)
    return np.concatenate([np.cos(a), np.sin(a)]).astype(np.float32)


# ---- the Llama graph (src/qwen.rs:1177-1528, dense branch) ---------------------------------------------
@dataclass
class LlamaConfig:
    n_layers: int
    h: int
    nh: int
    nkv: int
    hd: int
    inter: int
    vocab: int
    eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_interleaved: bool = True   # GGUF checkpoints (src/config.rs:926)

    @property
    def scale(self) -> float:
        return float(np.float32(1.0) / np.sqrt(np.float32(self.hd)))


def llama_graph(cfg: LlamaConfig, layers: list, final_norm: np.ndarray, head, rank: int = 0, world: int = 1, prefill: bool = False) -> Graph:
    """``layers``: per layer a dict with device weights ``q k v o gate up down`` and f32 arrays ``ln_pre ln_post``.
    Ten ops per layer (norm, q, k, v, qk-rope, attend, o, norm, gate+up pair, down), then the final norm and the head.

    ``world > 1`` builds rank ``rank``'s graph of a tensor-parallel plan: every weight is this rank's ROW shard
    (``shard_rows``: q / k / v by head, o / gate / up / down / head by equal row ranges), activations are replicated,
    and an exchange follows every sharded product whose output the next op needs in full (attention outputs, both
    residual updates, the MLP activations, the logits). Every output row is computed by the same kernel over the
    same inputs as on one GPU, so the results are bit-identical to the single-GPU plan.

    ``prefill``: the graph of a prefill plan, which ends at the final norm (no head, no logits: ``src/model_gpu.rs:398-400``)."""
    g = Graph()
    h, hd = cfg.h, cfg.hd
    assert cfg.nh % world == 0 and cfg.nkv % world == 0 and h % (32 * world) == 0 and cfg.inter % (32 * world) == 0 and cfg.vocab % (32 * world) == 0
    nh, nkv = cfg.nh // world, cfg.nkv // world          # this rank's heads
    qw = nh * hd
    x = g.buf(h)
    hn = g.buf(h)
    qkv = g.buf(qw + 2 * nkv * hd)
    qo = g.buf(nh * hd)
    att = g.buf(cfg.nh * hd)
    act = g.buf(cfg.inter)
    act2 = g.buf(cfg.inter)
    hidden = g.buf(h)
    logits = g.buf(1 if prefill else cfg.vocab)   # a prefill graph has no head (src/model_gpu.rs:77)
    g.input, g.n_input = x, h
    g.hidden, g.n_hidden = hidden, h
    g.rope_halves = [hd // 2]
    hs, ins, vs = h // world, cfg.inter // world, cfg.vocab // world   # row shares
    for L in layers:
        slot = len(g.kv)
        g.kv.append((nkv, hd))
        g.norm(x, hn, L["ln_pre"], h, cfg.eps)
        g.linear(L["q"], hn, qkv)
        g.linear(L["k"], hn, qkv.at(qw))
        g.linear(L["v"], hn, qkv.at(qw + nkv * hd))
        g.qk_rope(qkv, qo, slot, nh, nkv, hd, hd // 2, qw, qw + nkv * hd, cfg.rope_interleaved, cfg.eps)
        g.attend(qo, att.at(rank * qw), slot, nh, nkv, hd, cfg.scale)
        if world > 1:
            g.exchange(att, cfg.nh * hd)
        g.linear(L["o"], att, x.at(rank * hs), MODE_ADD)
        if world > 1:
            g.exchange(x, h)
        g.norm(x, hn, L["ln_post"], h, cfg.eps)
        if L["gate"].fmt == L["up"].fmt:   # pairable (src/gpu_decode.rs pairable)
            g.linear(L["gate"], hn, act.at(rank * ins), MODE_SILU_PAIR, dev2=L["up"])
        else:
            g.linear(L["gate"], hn, act2.at(rank * ins))
            g.linear(L["up"], hn, act.at(rank * ins))
            g.glu(act2.at(rank * ins), act.at(rank * ins), act.at(rank * ins), ins)
        if world > 1:
            g.exchange(act, cfg.inter)
        g.linear(L["down"], act, x.at(rank * hs), MODE_ADD)
        if world > 1:
            g.exchange(x, h)
    g.norm(x, hidden, final_norm, h, cfg.eps)
    if prefill:
        return g
    g.linear(head, hidden, logits.at(rank * vs))
    if world > 1:
        g.exchange(logits, cfg.vocab)
    g.logits = (logits, cfg.vocab)
    return g


def shard_llama(be, layers: list, head, cfg: LlamaConfig, rank: int, world: int):
    """Row shards of uploaded full matrices for rank ``rank`` (views into the same uploads): q / k / v by head, the rest
    by equal row ranges. Returns (layers, head) for ``llama_graph(..., rank, world)``."""
    def rows(dev, n):
        per = n // world
        return be.shard_rows(dev, rank * per, (rank + 1) * per)

    out = []
    for L in layers:
        S = {"ln_pre": L["ln_pre"], "ln_post": L["ln_post"]}
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            S[name] = rows(L[name], L[name].n_out)
        out.append(S)
    return out, rows(head, head.n_out)
