"""Whole-decoder-block forward and backward in two native calls.

A pre-norm decoder block is a fixed sequence of about a dozen kernel launches forward and two dozen
backward. Issued op by op from Python (one ``autograd.Function`` and one foreign call per launch)
the host needs longer to enqueue them than the GPU needs to run them. ``run`` hands the whole
sequence to the library's block runner (``csrc/block/block.cu``): Python allocates the outputs and
one activation arena, fills three small structs and makes one call; autograd sees one node per
block. The kernels, their order and their arguments are those of the op-by-op path, so both paths
produce the same numbers.

Taken for blocks whose projections are plain bf16 ``Linear`` layers (fused, or separate) or LoRA
wrappers around them, without biases. Tensor-parallel blocks on a token-sharded stream (sequence
parallelism with the fused all-gather / reduce-scatter GEMMs, fused QKV and gate-up weights, packed
batches) are taken too: the runner then issues the gathered and the reduced GEMMs and their device
barriers itself, on the symmetric buffers of the group's ``SPState``, in the order the op-by-op
path uses. Everything else (all-reduce tensor parallelism, FP8 / NF4 layers, Gemma's sandwich
norms, selective activation checkpointing, CPU tensors) keeps the op-by-op path.

Replaces the Python block of the reference (lset/models/decoder/qwen3/block.py:23-68).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _ac
from . import _native as nv
from ._grads import main_grad_of
from .norm import scratch
from .runtime_options import enabled, options as _rt

_vp, _fp, _ip = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p


class LbLinear(ctypes.Structure):
    _fields_ = [("w", _vp), ("wgrad", _fp), ("lora_a", _vp), ("lora_b", _vp),
                ("lora_a_grad", _fp), ("lora_b_grad", _fp), ("ldw", ctypes.c_longlong),
                ("n_out", ctypes.c_int), ("k_in", ctypes.c_int), ("lora_r", ctypes.c_int),
                ("lora_scale", ctypes.c_float)]


class LbProjection(ctypes.Structure):
    _fields_ = [("part", LbLinear * 3), ("n", ctypes.c_int), ("width", ctypes.c_int)]


class LbBlockDesc(ctypes.Structure):
    _fields_ = [("H", ctypes.c_int), ("Hq", ctypes.c_int), ("Hk", ctypes.c_int),
                ("hd", ctypes.c_int), ("I", ctypes.c_int), ("causal", ctypes.c_int),
                ("act_kind", ctypes.c_int), ("qk_norm", ctypes.c_int), ("eps", ctypes.c_float),
                ("w_off", ctypes.c_float), ("softmax_scale", ctypes.c_float),
                ("ln1_w", _vp), ("ln1_wgrad", _fp), ("ln2_w", _vp), ("ln2_wgrad", _fp),
                ("qn_w", _vp), ("qn_wgrad", _fp), ("kn_w", _vp), ("kn_wgrad", _fp),
                ("qkv", LbProjection), ("gate_up", LbProjection), ("o_proj", LbLinear),
                ("down", LbLinear)]


class LbStreamCtx(ctypes.Structure):
    _fields_ = [("T", ctypes.c_int), ("packed", ctypes.c_int), ("cos", _fp), ("sin", _fp),
                ("pos", _vp), ("pos_i64", ctypes.c_int), ("seq_start", _ip), ("seq_end", _ip),
                ("plan_q", _ip), ("cap_q", ctypes.c_int), ("plan_kv", _ip),
                ("cap_kv", ctypes.c_int), ("status", _ip), ("norm_scratch", _fp),
                ("rope_scratch", _fp), ("wg_tmp", _fp), ("stream", _vp)]


class LbTpCtx(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows", ctypes.c_int),
                ("reserved", ctypes.c_int), ("ag_peers", _vp * 2), ("ag_local", _vp * 2),
                ("ag_flags", _vp), ("ag_counter", _vp), ("rs_peers", _vp * 2),
                ("rs_local", _vp * 2), ("pads", _vp), ("bar_limit_ns", ctypes.c_ulonglong),
                ("ag_epoch", ctypes.c_uint), ("ag_calls", ctypes.c_uint),
                ("rs_epoch", ctypes.c_uint), ("bar_epoch", ctypes.c_uint)]


class LbBlockIO(ctypes.Structure):
    _fields_ = [("branch", _vp), ("residual", _vp), ("out", _vp), ("res_out", _vp),
                ("saved", _vp), ("d_out", _vp), ("d_res_out", _vp), ("dx", _vp), ("work", _vp),
                ("tp", _vp)]


_lib = None
calls = {"dp": 0, "tp": 0}   # block forwards taken by the runner, by stream layout (for tests)


def _library():
    global _lib
    if _lib is None:
        lib = nv.load()
        lib.lb_block_saved_bytes.restype = ctypes.c_size_t
        lib.lb_block_work_bytes.restype = ctypes.c_size_t
        for fn in (lib.lb_block_fwd, lib.lb_block_bwd):
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.lb_block_saved_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_void_p]
        lib.lb_block_work_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.lb_block_fwd_launches.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                              ctypes.c_void_p]
        lib.lb_block_bwd_launches.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        _lib = lib
    return _lib


_arenas = {}


def _arena_size(nbytes: int) -> int:
    """``nbytes`` rounded up to the next size of a geometric series (eight sizes per octave, at
    most 12.5 % more). Packed batches differ in token count from step to step; with exact sizes
    every batch longer than all before it makes the caching allocator ask the driver for one new
    block per decoder block (a stall of up to several hundred milliseconds on a busy host), with
    rounded sizes that happens a few times at the start of a run and then no more."""
    if nbytes <= (1 << 20):
        return max(nbytes, 1)
    top = 1 << (nbytes.bit_length() - 1)       # largest power of two <= nbytes
    step = top >> 3
    return (nbytes + step - 1) // step * step


def _work_arena(nbytes: int, device) -> torch.Tensor:
    """Temporary storage of the block backward: one buffer per device, grown on demand. Blocks run
    their backward one after the other on the same stream, so they share it."""
    t = _arenas.get(device)
    if t is None or t.numel() < nbytes:
        t = torch.empty(_arena_size(nbytes), dtype=torch.uint8, device=device)
        _arenas[device] = t
    return t


# --------------------------------------------------------------------------- eligibility
def _plain_linear(m) -> bool:
    from ..models.layers import Linear

    return (type(m) is Linear and m.bias is None and "forward" not in m.__dict__
            and not hasattr(m, "_tp_kind") and m.weight.dtype == torch.bfloat16
            and m.weight.is_cuda and m.weight.stride(-1) == 1)


def _sp_linear(m, kind: str, st) -> bool:
    """A bias-free bf16 ``Linear`` that ``apply_tp`` wrapped for the token-sharded stream."""
    from ..models.layers import Linear

    return (type(m) is Linear and m.bias is None and getattr(m, "_tp_kind", None) == kind
            and getattr(m, "_sp_state", None) is st and m.weight.dtype == torch.bfloat16
            and m.weight.is_cuda and m.weight.stride(-1) == 1)


def _linear_parts(m):
    """``(weight, lora_A weight or None, lora_B weight or None, scale)`` for a supported projection
    module, else None."""
    if _plain_linear(m):
        return m.weight, None, None, 0.0
    base = getattr(m, "base_linear", None)
    if base is not None and hasattr(m, "lora_A") and _plain_linear(base):
        a, b = m.lora_A, m.lora_B
        drop = getattr(m, "dropout", None)
        if (_plain_linear(a) and _plain_linear(b) and m.r % 8 == 0
                and (isinstance(drop, torch.nn.Identity) or not m.training)):
            return base.weight, a.weight, b.weight, float(m.scale)
    return None


class BlockPlan:
    """What the runner needs to know about one ``DecoderBlock``: which tensors feed which field of
    the descriptor. Pointers are re-read on every call (parameters may be re-homed into flat
    buffers after the plan was made)."""

    def __init__(self, block):
        att, mlp, tr = block.self_attn, block.mlp, block.traits
        self.ok = False
        self.signature = self._signature(block)
        if tr.sandwich_norms or att.head_dim not in (64, 128):
            return
        if att.num_heads % att.num_kv_heads or (att.num_heads // att.num_kv_heads) not in (1, 2, 4, 8):
            return
        qkv_mods = [att.qkv_proj] if att.fused_qkv else [att.q_proj, att.k_proj, att.v_proj]
        gu_mods = [mlp.gate_up_proj] if mlp.fused_gate_up else [mlp.gate_proj, mlp.up_proj]
        mods = qkv_mods + [att.o_proj] + gu_mods + [mlp.down_proj]
        # tensor parallelism on a token-sharded stream: every projection carries the group's state
        self.sp = getattr(att.o_proj, "_sp_state", None)
        if self.sp is not None:
            kinds = ("colwise", "rowwise", "colwise", "rowwise")
            if len(mods) != 4 or not all(_sp_linear(m, k, self.sp) for m, k in zip(mods, kinds)):
                return
            parts = [(m.weight, None, None, 0.0) for m in mods]
        else:
            parts = [_linear_parts(m) for m in mods]
        if any(p is None for p in parts):
            return
        self.qkv, self.o = parts[:len(qkv_mods)], parts[len(qkv_mods)]
        self.gate_up, self.down = parts[len(qkv_mods) + 1:-1], parts[-1]
        self.ln1, self.ln2 = block.input_layernorm, block.post_attention_layernorm
        self.qn = att.q_norm.weight if att.q_norm is not None else None
        self.kn = att.k_norm.weight if att.k_norm is not None else None
        hd = att.head_dim
        H = self.ln1.weight.shape[0]
        width = sum(p[0].shape[0] for p in self.qkv)
        if width % ((att.num_heads // att.num_kv_heads + 2) * hd):
            return
        Hk = width // ((att.num_heads // att.num_kv_heads + 2) * hd)
        Hq = Hk * (att.num_heads // att.num_kv_heads)
        I = sum(p[0].shape[0] for p in self.gate_up) // 2
        if H % 8 or I % 8 or self.down[0].shape[1] != I or self.o[0].shape[1] != Hq * hd:
            return
        if len(self.gate_up) == 2 and self.gate_up[0][0].shape[0] != I:
            return
        if len(self.qkv) == 3 and [p[0].shape[0] for p in self.qkv] != [Hq * hd, Hk * hd, Hk * hd]:
            return
        for w in (self.ln1.weight, self.ln2.weight, self.qn, self.kn):
            if w is not None and (w.dtype != torch.bfloat16 or not w.is_cuda):
                return
        d = LbBlockDesc()
        d.H, d.Hq, d.Hk, d.hd, d.I = H, Hq, Hk, hd, I
        d.causal = int(att.causal)
        d.act_kind = {"swiglu": 0, "geglu": 1}[mlp.kind]
        d.qk_norm = int(self.qn is not None)
        d.eps, d.w_off = float(self.ln1.eps), float(self.ln1.w_off)
        d.softmax_scale = float(att.softmax_scale if att.softmax_scale is not None
                                else 1.0 / math.sqrt(hd))
        d.qkv.n, d.qkv.width = len(self.qkv), width
        d.gate_up.n, d.gate_up.width = len(self.gate_up), 2 * I
        self.desc = d
        self.rope = (hd, att.rope_theta, att.rope_scaling)
        # every trainable tensor, in the order the autograd node lists them
        self.params = []
        for w in (self.ln1.weight, self.ln2.weight, self.qn, self.kn):
            if w is not None:
                self.params.append(w)
        for p in self.qkv + [self.o] + self.gate_up + [self.down]:
            self.params.extend(t for t in p[:3] if t is not None)
        self._launches = {}
        self.ok = True

    @staticmethod
    def _signature(block):
        """Changes when a projection is wrapped, replaced, moved or cast after the plan was made."""
        att, mlp = block.self_attn, block.mlp
        mods = (([att.qkv_proj] if att.fused_qkv else [att.q_proj, att.k_proj, att.v_proj])
                + [att.o_proj]
                + ([mlp.gate_up_proj] if mlp.fused_gate_up else [mlp.gate_proj, mlp.up_proj])
                + [mlp.down_proj])
        return tuple((id(m), "forward" in m.__dict__, id(getattr(m, "_sp_state", None)),
                      m.weight.dtype, m.weight.device, m.training) for m in mods)

    def still_valid(self, block) -> bool:
        return self.signature == self._signature(block)

    # ------------------------------------------------------------------ descriptor
    @staticmethod
    def _fill_linear(dst: LbLinear, part, grads) -> None:
        w, a, b, scale = part
        dst.w = w.data_ptr()
        dst.ldw = w.stride(0)
        dst.n_out, dst.k_in = w.shape
        dst.wgrad = grads.get(id(w))
        if a is not None:
            dst.lora_a, dst.lora_b = a.data_ptr(), b.data_ptr()
            dst.lora_a_grad, dst.lora_b_grad = grads.get(id(a)), grads.get(id(b))
            dst.lora_r, dst.lora_scale = a.shape[0], scale
        else:
            dst.lora_a = dst.lora_b = dst.lora_a_grad = dst.lora_b_grad = None
            dst.lora_r, dst.lora_scale = 0, 0.0

    def fill(self, grads: dict) -> LbBlockDesc:
        """Refresh every pointer. ``grads`` maps ``id(param)`` to the address of its fp32 gradient
        accumulator (absent = no weight gradient wanted)."""
        d = self.desc
        d.ln1_w, d.ln1_wgrad = self.ln1.weight.data_ptr(), grads.get(id(self.ln1.weight))
        d.ln2_w, d.ln2_wgrad = self.ln2.weight.data_ptr(), grads.get(id(self.ln2.weight))
        if self.qn is not None:
            d.qn_w, d.qn_wgrad = self.qn.data_ptr(), grads.get(id(self.qn))
            d.kn_w, d.kn_wgrad = self.kn.data_ptr(), grads.get(id(self.kn))
        for i, p in enumerate(self.qkv):
            self._fill_linear(d.qkv.part[i], p, grads)
        for i, p in enumerate(self.gate_up):
            self._fill_linear(d.gate_up.part[i], p, grads)
        self._fill_linear(d.o_proj, self.o, grads)
        self._fill_linear(d.down, self.down, grads)
        return d


def plan_of(block):
    plan = block.__dict__.get("_lb_plan")
    if plan is None or not plan.still_valid(block):
        plan = BlockPlan(block)
        block.__dict__["_lb_plan"] = plan
    return plan if plan.ok else None


def usable(block, branch, ctx) -> bool:
    """True when this call can go through the block runner."""
    if not (branch.is_cuda and branch.dtype == torch.bfloat16 and branch.dim() == 2):
        return False
    if _ac._active is not None or not enabled("block_runner") or _rt.attention_backend == "sdpa":
        return False
    for name in ("fused_rmsnorm", "fused_residual_rmsnorm", "fused_qk_norm_rope"):
        if not enabled(name):
            return False
    plan = plan_of(block)
    if plan is None:
        return False
    if plan.sp is None:
        if ctx.pos.shape[0] != branch.shape[0]:  # a token-sharded stream needs the group's state
            return False
    elif not _sp_ready(plan.sp, branch, ctx):
        return False
    if torch.is_grad_enabled() and plan.desc.hd > 128:
        return False
    return True


# --------------------------------------------------------------------------- token-sharded stream
def _sp_ready(st, branch, ctx) -> bool:
    """The runner drives the fused tensor-parallel GEMMs only on peer memory with bf16
    accumulators and the device barrier, for packed batches."""
    st.bind(branch.device)
    if not (st.fused and st.rs_bf16 and enabled("tp_block_runner")):
        return False
    if ctx.plan.cu_seqlens is None or branch.shape[0] * st.world < ctx.pos.shape[0]:
        return False
    return st.token().pad is not None


def _tp_struct(st, rows: int, H: int):
    """The group's symmetric buffers and counters as the runner's struct, plus what to advance
    after the call. Buffers are created (a rendezvous of the group) on first use or growth; every
    rank gets here with the same shapes."""
    buf, rs, tok = st.ag_buf(rows, H), st.rs_buf(rows, H), st.token()
    fl = buf.flags(rows)
    t = LbTpCtx()
    t.world, t.rank, t.rows = st.world, st.rank, rows
    keep = []
    for i in range(2):
        a, b = buf.x_sym[i].c_ptr_array(), rs.slot_ptrs(i, rows, H)
        keep += [a, b]
        t.ag_peers[i] = ctypes.cast(a, ctypes.c_void_p)
        t.rs_peers[i] = ctypes.cast(b, ctypes.c_void_p)
        t.ag_local[i] = buf.x_sym[i].local.data_ptr()
        t.rs_local[i] = rs.acc[i].local.data_ptr()
    t.ag_flags, t.ag_counter = fl[0].data_ptr(), buf.counter.data_ptr()
    pads = tok.pad.c_ptr_array()
    keep.append(pads)
    t.pads = ctypes.cast(pads, ctypes.c_void_p)
    t.bar_limit_ns = tok.limit_ns
    t.ag_epoch, t.ag_calls = st._ag_epoch[H], fl[1]
    t.rs_epoch, t.bar_epoch = rs.epoch, tok.epoch
    t._keep = keep
    return t, (st, H, fl, rs, tok)


def _tp_advance(state) -> None:
    """Each runner call makes two uses of the publication area and of the accumulators and passes
    four barriers (see ``LbTpCtx`` in csrc/block/block.h)."""
    st, H, fl, rs, tok = state
    st._ag_epoch[H] += 2
    fl[1] += 2
    rs.epoch += 2
    tok.epoch += 4


# --------------------------------------------------------------------------- stream context
def _stream_struct(ctx, plan: BlockPlan, device) -> LbStreamCtx:
    """The per-forward struct, cached on the Python stream context (all blocks share it)."""
    d = plan.desc
    key = ("_lb", d.hd, d.Hq // d.Hk, plan.rope[1], id(plan.rope[2]))
    hit = ctx.tables.get(key)
    if hit is not None:
        return hit
    lib = _library()
    cos, sin = ctx.rope(*plan.rope)
    ap = ctx.plan
    ptq, capq = ap.tiles(128 // (d.Hq // d.Hk))
    ptk, capk = ap.tiles(128)
    s = LbStreamCtx()
    s.T, s.packed = int(ctx.pos.shape[0]), int(ap.cu_seqlens is not None)
    s.cos, s.sin = cos.data_ptr(), sin.data_ptr()
    s.pos, s.pos_i64 = ctx.pos.data_ptr(), int(ctx.pos.dtype == torch.int64)
    s.seq_start, s.seq_end = ap.seq_start.data_ptr(), ap.seq_end.data_ptr()
    s.plan_q, s.cap_q, s.plan_kv, s.cap_kv = ptq.data_ptr(), capq, ptk.data_ptr(), capk
    s.status = nv.status_word(device).data_ptr()
    s.norm_scratch = scratch("norm_bwd", lib.lb_norm_bwd_partial_rows() * d.H, device).data_ptr()
    s.rope_scratch = scratch("rope_bwd", lib.lb_rope_bwd_partial_rows() * 2 * d.hd,
                             device).data_ptr()
    s.wg_tmp = scratch("qk_norm_wgrad", 2 * d.hd, device).data_ptr()
    s.stream = 0
    # keep the tensors the struct points to alive as long as the struct
    s._keep = (cos, sin, ctx.pos, ap, ptq, ptk)
    ctx.tables[key] = s
    return s


# --------------------------------------------------------------------------- autograd node
class _BlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, branch, residual, plan, sctx, stream_ctx, *params):
        lib = _library()
        dev = branch.device
        d = plan.fill({})
        T, H = branch.shape
        branch = branch if branch.is_contiguous() else branch.contiguous()
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        has_res = residual is not None
        # token-sharded stream: T is this rank's row count and the struct names the group's buffers
        tp, tp_state = _tp_struct(plan.sp, T, H) if plan.sp is not None else (None, None)
        tp_ptr = ctypes.addressof(tp) if tp is not None else None
        nbytes = lib.lb_block_saved_bytes(ctypes.addressof(d), T, int(has_res), tp_ptr)
        saved = torch.empty(_arena_size(nbytes), dtype=torch.uint8, device=dev)
        out = torch.empty(T, H, dtype=branch.dtype, device=dev)
        res_out = torch.empty(T, H, dtype=branch.dtype, device=dev)
        io = LbBlockIO()
        io.tp = tp_ptr
        io.branch, io.residual = branch.data_ptr(), (residual.data_ptr() if has_res else None)
        io.out, io.res_out, io.saved = out.data_ptr(), res_out.data_ptr(), saved.data_ptr()
        sctx.stream = nv.stream_ptr()
        rc = lib.lb_block_fwd(ctypes.addressof(d), ctypes.addressof(sctx), ctypes.addressof(io))
        if rc != 0:
            nv.check_rc(rc, "lb_block_fwd")
        if tp is not None:
            _tp_advance(tp_state)
        calls["tp" if tp is not None else "dp"] += 1
        n = plan._launches.get(("f", sctx.packed))
        if n is None:
            n = lib.lb_block_fwd_launches(ctypes.addressof(d), ctypes.addressof(sctx), int(has_res),
                                          tp_ptr)
            plan._launches[("f", sctx.packed)] = n
        nv.count_launch(n)
        ctx.save_for_backward(branch, residual, saved, res_out)
        ctx.plan, ctx.sctx, ctx.stream_ctx = plan, sctx, stream_ctx
        return out, res_out

    @staticmethod
    def backward(ctx, d_out, d_res_out):
        lib = _library()
        branch, residual, saved, res_out = ctx.saved_tensors
        plan, sctx = ctx.plan, ctx.sctx
        dev = branch.device
        T, H = branch.shape
        if d_out is None:
            d_out = torch.zeros(T, H, dtype=branch.dtype, device=dev)
        d_out = d_out if d_out.is_contiguous() else d_out.contiguous()
        if d_res_out is not None and not d_res_out.is_contiguous():
            d_res_out = d_res_out.contiguous()
        # weight gradients go straight into the sharding runtime's fp32 accumulators; a parameter
        # without one gets a temporary that is returned to autograd
        grads, temps = {}, []
        for p in plan.params:
            if not p.requires_grad:
                temps.append(None)
                continue
            mg = main_grad_of(p)
            if mg is None:
                mg = torch.zeros(p.shape, dtype=torch.float32, device=dev)
                temps.append(mg)
            else:
                temps.append(None)
            grads[id(p)] = mg.data_ptr()
        d = plan.fill(grads)
        tp, tp_state = _tp_struct(plan.sp, T, H) if plan.sp is not None else (None, None)
        tp_ptr = ctypes.addressof(tp) if tp is not None else None
        work = _work_arena(lib.lb_block_work_bytes(ctypes.addressof(d), T, tp_ptr), dev)
        dx = torch.empty(T, H, dtype=branch.dtype, device=dev)
        io = LbBlockIO()
        io.tp = tp_ptr
        io.branch = branch.data_ptr()
        io.residual = residual.data_ptr() if residual is not None else None
        io.res_out, io.saved = res_out.data_ptr(), saved.data_ptr()
        io.d_out = d_out.data_ptr()
        io.d_res_out = d_res_out.data_ptr() if d_res_out is not None else None
        io.dx, io.work = dx.data_ptr(), work.data_ptr()
        sctx.stream = nv.stream_ptr()
        rc = lib.lb_block_bwd(ctypes.addressof(d), ctypes.addressof(sctx), ctypes.addressof(io))
        if rc != 0:
            nv.check_rc(rc, "lb_block_bwd")
        if tp is not None:
            _tp_advance(tp_state)
        key = ("b", sctx.packed, len(grads))
        n = plan._launches.get(key)
        if n is None:
            n = lib.lb_block_bwd_launches(ctypes.addressof(d), ctypes.addressof(sctx), tp_ptr)
            plan._launches[key] = n
        nv.count_launch(n)
        pgrads = tuple(None if t is None else t.to(p.dtype) for t, p in zip(temps, plan.params))
        return (dx, dx if residual is not None else None, None, None, None) + pgrads


def run(block, branch, residual, ctx):
    """``(mlp_out, residual_out)`` of one decoder block, as ``DecoderBlock.forward`` returns them."""
    plan = plan_of(block)
    sctx = _stream_struct(ctx, plan, branch.device)
    return _BlockFn.apply(branch, residual, plan, sctx, ctx, *plan.params)
