"""Expert-parallel MoE layers.

``FusedEPMoE`` runs the routed experts of one MoE layer across the ranks of a group with the
single-kernel dispatch -> grouped SwiGLU GEMM -> weighted combine of csrc/moe_kernels.cu:
token rows are pushed into the owning rank's expert-sorted buffer over NVLink, the tcgen05
grouped GEMMs start per expert as its rows arrive, and the down-projection epilogue adds the
weighted result straight into the token owner's output row. ``NcclEPMoE`` is the library
baseline with the same math: ``all_to_all_single`` dispatch, per-expert GEMMs, ``all_to_all_single``
combine (jax_gpt_b200/models/qwen35/moe.py:expert_forward_ep).

The reference's expert parallelism replicates the tokens and sums full outputs with one psum
(jax_gpt/models/qwen35/moe.py:117-222).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _ext
from ..comm.symm import Communicator


class FusedEPMoE:
    """Buffers and launch logic of the fused expert-parallel forward for a fixed problem size.

    ``tokens``: tokens owned by every rank; ``n_experts``: global expert count (experts
    ``[r * E/W, (r+1) * E/W)`` live on rank r); ``cap_factor``: receive-buffer rows as a multiple
    of the balanced load ``tokens * top_k`` (the worst case is ``world``).
    """

    def __init__(self, comm: Communicator, tokens: int, d_model: int, inter: int, n_experts: int, top_k: int,
                 cap_factor: Optional[float] = None, training: bool = False):
        self.comm = comm
        W = comm.world
        assert n_experts % W == 0 and d_model % 256 == 0 and inter % 128 == 0
        self.tokens, self.D, self.I, self.E, self.k = tokens, d_model, inter, n_experts, top_k
        self.e_local = n_experts // W
        cap_factor = float(W) if cap_factor is None else cap_factor
        # every expert's region is padded to a multiple of 64 rows
        self.cap_rows = (int(tokens * top_k * cap_factor) + 64 * self.e_local + 127) // 128 * 128
        self.training = training
        self.launch_token = 0    # identifies the forward launch whose state sits in the buffers
        dev = comm.device
        self.recv_x = comm.alloc(self.cap_rows * d_model, torch.bfloat16, zero=True)
        self.recv_meta = comm.alloc(self.cap_rows, torch.int32)
        self.recv_w = comm.alloc(self.cap_rows, torch.float32)
        self.counts_all = comm.alloc(W * n_experts, torch.int32)
        self.arrive = comm.alloc(max(self.e_local, 32), torch.int32)
        self.out_acc = comm.alloc(tokens * d_model, torch.float32)
        self.act = torch.zeros(self.cap_rows, inter, device=dev, dtype=torch.bfloat16)
        self.arrive_target = torch.zeros(self.e_local, device=dev, dtype=torch.int32)
        self.act_ready = torch.zeros(self.cap_rows // 128 + self.e_local + 1, device=dev, dtype=torch.int32)  # + tile counter
        self.slot_out = torch.zeros(tokens * top_k, device=dev, dtype=torch.int32)
        self.rows_out = torch.zeros(self.e_local, device=dev, dtype=torch.int32)
        self.my_counts = torch.zeros(n_experts, device=dev, dtype=torch.int32)
        self.pos = torch.zeros(tokens * top_k, device=dev, dtype=torch.int32)
        if training:
            self.gu = torch.zeros(self.cap_rows, 2 * inter, device=dev, dtype=torch.bfloat16)
            self.dgu = torch.zeros(self.cap_rows, 2 * inter, device=dev, dtype=torch.bfloat16)
            self.recv_dy = comm.alloc(self.cap_rows * d_model, torch.bfloat16, zero=True)
            self.dx_acc = comm.alloc(tokens * d_model, torch.float32)
            self.dw_out = comm.alloc(tokens * top_k, torch.float32)
            self.dw_rows = torch.zeros(self.cap_rows, device=dev, dtype=torch.float32)
            self.gu_ready = torch.zeros(self.cap_rows // 128 + self.e_local + 1, device=dev, dtype=torch.int32)  # + tile counter
            self.expert_done = torch.zeros(self.e_local, device=dev, dtype=torch.int32)
        else:
            self.gu = None
        dist.barrier(comm.group)

    def backward(self, x, dout, weights, idx, params, grads):
        """Gradients of the LAST ``forward`` call (same x, routing and params): the dispatched x rows,
        their slots, the activations and the pre-activations of that launch are reused in place, only the
        routing-weighted ``dout`` rows travel. ``grads`` holds fp32 ``gate_proj`` / ``up_proj`` /
        ``down_proj`` buffers that are ACCUMULATED into. Returns (dx (tokens, D) fp32, dweights (tokens, k) fp32)."""
        assert self.training, "construct FusedEPMoE(training=True) to keep what backward needs"
        ops = _ext.ops()
        c = self.comm
        idx32 = idx.to(torch.int32).contiguous().view(-1)
        w32 = weights.to(torch.float32).contiguous().view(-1)
        self.dx_acc.tensor.zero_()   # my_counts / pos are the forward launch's: the slots must not change
        ops.ep_moe_backward(c.world, c.rank, self.k, self.e_local, self.cap_rows, x.contiguous(), dout.contiguous(),
                            idx32, w32, self.pos, self.my_counts, self.recv_x.peer_ptrs, self.recv_dy.peer_ptrs,
                            self.recv_meta.peer_ptrs, self.recv_w.peer_ptrs, self.counts_all.peer_ptrs,
                            self.arrive.peer_ptrs, self.dx_acc.peer_ptrs, self.dw_out.peer_ptrs, c.ctrl.peer_ptrs,
                            self.act, self.gu, self.dgu, self.dw_rows, self.arrive_target, self.gu_ready,
                            self.expert_done, self.slot_out, self.rows_out, params["gate_proj"], params["up_proj"],
                            params["down_proj"], grads["gate_proj"], grads["up_proj"], grads["down_proj"],
                            c.wait_seconds)
        return self.dx_acc.tensor.view(self.tokens, self.D), self.dw_out.tensor.view(self.tokens, self.k)

    def forward(self, x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, params: dict,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x (tokens, D) bf16; weights / idx (tokens, k); params hold this rank's experts stacked:
        gate_proj / up_proj (E_local, D, I), down_proj (E_local, I, D). Returns (tokens, D) fp32."""
        ops = _ext.ops()
        c = self.comm
        idx32 = idx.to(torch.int32).contiguous().view(-1)
        w32 = weights.to(torch.float32).contiguous().view(-1)
        ops.moe_prepare(idx32, self.my_counts, self.pos)
        self.launch_token += 1
        self.out_acc.tensor.zero_()
        ops.ep_moe_forward(c.world, c.rank, self.k, self.e_local, self.cap_rows, x.contiguous(), idx32, w32, self.pos,
                           self.my_counts, self.recv_x.peer_ptrs, self.recv_meta.peer_ptrs, self.recv_w.peer_ptrs,
                           self.counts_all.peer_ptrs, self.arrive.peer_ptrs, self.out_acc.peer_ptrs, c.ctrl.peer_ptrs,
                           self.act, self.arrive_target, self.act_ready, self.slot_out, self.rows_out,
                           params["gate_proj"], params["up_proj"], params["down_proj"], c.wait_seconds, self.gu)
        res = self.out_acc.tensor.view(self.tokens, self.D)
        if out is not None:
            out.copy_(res)
            return out
        return res


def quantize_expert_weights_fp8(params: dict) -> dict:
    """Stacked bf16 expert weights (gate_proj / up_proj (E, D, I), down_proj (E, I, D)) -> what the FP8
    kernel reads: K-major e4m3 bytes with power-of-two 128 x 128 block scales, and the packed UE8M0
    scale chunks (csrc/moe_kernels.cuh: EpMoeFp8Args)."""
    from ..ops.fp8 import fp8_quant_128x128
    gate, up, down = params["gate_proj"], params["up_proj"], params["down_proj"]
    E, D, I = gate.shape
    dev = gate.device

    def q(w):  # (E, K, N) -> bytes (E, N, K), exponents (E, N/128, K/128)
        qs, es = [], []
        for e in range(w.shape[0]):
            qe, se = fp8_quant_128x128(w[e].t().contiguous().to(torch.bfloat16), pow2=True)
            qs.append(qe.view(torch.uint8))
            es.append((torch.log2(se.float()).round() + 127).clamp(1, 254).to(torch.uint8))
        return torch.stack(qs), torch.stack(es)

    gq, ge = q(gate)
    uq, ue = q(up)
    dq, de = q(down)
    # GEMM 1 chunk: rows 0-63 of the B tile are gate rows, 64-127 up rows -> 32-row groups (gate, gate, up, up)
    grp = torch.stack([ge, ge, ue, ue], dim=-1)                                   # (E, I/128, D/128, 4)
    sfb1 = grp[:, :, :, None, :, None].expand(E, I // 128, D // 128, 32, 4, 4).reshape(E, I // 128, D // 128, 512)
    sfb2 = de[:, :, :, None].expand(E, D // 128, I // 128, 512)
    return {"gate_q": gq.contiguous(), "up_q": uq.contiguous(), "down_q": dq.contiguous(),
            "sfb1": sfb1.contiguous(), "sfb2": sfb2.contiguous(), "gate_e": ge, "up_e": ue, "down_e": de}


def fp8_moe_reference(x, weights, idx, qw_full: dict) -> torch.Tensor:
    """fp32 restatement of the FP8 kernel's arithmetic with ALL experts local: 1 x 128 power-of-two
    activation quantisation, de-quantised block-scaled weights, SwiGLU, re-quantised activation."""
    from ..ops.fp8 import fp8_quant_1x128_ref

    def deq(qb, eb):  # (N, K) bytes + (N/128, K/128) exponents -> fp32 (N, K)
        sc = torch.exp2(eb.float() - 127).repeat_interleave(128, 0).repeat_interleave(128, 1)
        return qb.view(torch.float8_e4m3fn).float() * sc

    def qdq(t):
        qv, sc = fp8_quant_1x128_ref(t, pow2=True)
        return (qv.float().view(t.shape[0], -1, 128) * sc[..., None]).view(t.shape)

    xq = qdq(x.float())
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    for e in idx.unique().tolist():
        tok, slot = (idx == e).nonzero(as_tuple=True)
        g = xq[tok] @ deq(qw_full["gate_q"][e], qw_full["gate_e"][e]).t()
        u = xq[tok] @ deq(qw_full["up_q"][e], qw_full["up_e"][e]).t()
        act = qdq(torch.nn.functional.silu(g) * u)
        y = act @ deq(qw_full["down_q"][e], qw_full["down_e"][e]).t()
        out.index_add_(0, tok, y * weights[tok, slot][:, None].float())
    return out


class FusedEPMoEFp8:
    """FP8 forward of the fused expert-parallel layer: e4m3 rows with power-of-two 1 x 128 scales on the
    wire and in the grouped GEMMs (tensor-core block scaling), weights pre-quantised with
    ``quantize_expert_weights_fp8``. Same constructor arguments as ``FusedEPMoE``."""

    def __init__(self, comm: Communicator, tokens: int, d_model: int, inter: int, n_experts: int, top_k: int,
                 cap_factor: Optional[float] = None):
        self.comm = comm
        W = comm.world
        assert n_experts % W == 0 and d_model % 256 == 0 and inter % 128 == 0
        self.tokens, self.D, self.I, self.E, self.k = tokens, d_model, inter, n_experts, top_k
        self.e_local = n_experts // W
        cap_factor = float(W) if cap_factor is None else cap_factor
        self.cap_rows = (int(tokens * top_k * cap_factor) + 128 * self.e_local + 127) // 128 * 128
        dev = comm.device
        u8 = torch.uint8
        self.recv_q = comm.alloc(self.cap_rows * d_model, u8, zero=True)
        self.recv_sf = comm.alloc((self.cap_rows // 128) * (d_model // 128) * 512, u8, zero=True)
        self.recv_meta = comm.alloc(self.cap_rows, torch.int32)
        self.recv_w = comm.alloc(self.cap_rows, torch.float32)
        self.counts_all = comm.alloc(W * n_experts, torch.int32)
        self.arrive = comm.alloc(max(self.e_local, 32), torch.int32)
        self.out_acc = comm.alloc(tokens * d_model, torch.float32)
        self.xq = torch.zeros(tokens, d_model, device=dev, dtype=u8)
        self.xe = torch.zeros(tokens, d_model // 128, device=dev, dtype=u8)
        self.act_q = torch.zeros(self.cap_rows, inter, device=dev, dtype=u8)
        self.act_sf = torch.full(((self.cap_rows // 128) * (inter // 128) * 512,), 127, device=dev, dtype=u8)
        self.arrive_target = torch.zeros(self.e_local, device=dev, dtype=torch.int32)
        self.act_ready = torch.zeros(self.cap_rows // 128 + self.e_local, device=dev, dtype=torch.int32)
        self.slot_out = torch.zeros(tokens * top_k, device=dev, dtype=torch.int32)
        self.rows_out = torch.zeros(self.e_local, device=dev, dtype=torch.int32)
        self.my_counts = torch.zeros(n_experts, device=dev, dtype=torch.int32)
        self.pos = torch.zeros(tokens * top_k, device=dev, dtype=torch.int32)
        dist.barrier(comm.group)

    def forward(self, x, weights, idx, qw: dict) -> torch.Tensor:
        """x (tokens, D) bf16; ``qw``: this rank's experts from ``quantize_expert_weights_fp8``. Returns fp32."""
        ops = _ext.ops()
        c = self.comm
        idx32 = idx.to(torch.int32).contiguous().view(-1)
        w32 = weights.to(torch.float32).contiguous().view(-1)
        ops.moe_prepare(idx32, self.my_counts, self.pos)
        self.out_acc.tensor.zero_()
        ops.ep_moe_forward_fp8(c.world, c.rank, self.k, self.e_local, self.cap_rows, x.contiguous(), idx32, w32, self.pos,
                               self.my_counts, self.xq, self.xe, self.recv_q.peer_ptrs, self.recv_sf.peer_ptrs,
                               self.recv_meta.peer_ptrs, self.recv_w.peer_ptrs, self.counts_all.peer_ptrs,
                               self.arrive.peer_ptrs, self.out_acc.peer_ptrs, c.ctrl.peer_ptrs, self.act_q, self.act_sf,
                               self.arrive_target, self.act_ready, self.slot_out, self.rows_out, qw["gate_q"],
                               qw["up_q"], qw["down_q"], qw["sfb1"], qw["sfb2"], c.wait_seconds)
        return self.out_acc.tensor.view(self.tokens, self.D)


class _FusedEPMoEFn(torch.autograd.Function):
    """Autograd node around one ``FusedEPMoE`` layer. Expert weights stay outside autograd: their fp32
    gradients are accumulated by the backward kernel straight into ``grads`` (main-grad convention)."""

    @staticmethod
    def forward(ctx, x, weights, idx, layer, params, grads):
        out = layer.forward(x, weights, idx, params)
        ctx.layer, ctx.params, ctx.grads = layer, params, grads
        ctx.token = layer.launch_token
        ctx.save_for_backward(x, weights, idx)
        return out.to(x.dtype)   # a copy: the symmetric accumulation buffer is reused by the next launch

    @staticmethod
    def backward(ctx, dout):
        x, weights, idx = ctx.saved_tensors
        layer = ctx.layer
        if layer.launch_token != ctx.token:
            # another MoE layer used the buffers since: recompute this layer's dispatch and activations
            layer.forward(x, weights, idx, ctx.params)
        dx, dw = layer.backward(x, dout.to(torch.bfloat16), weights, idx, ctx.params, ctx.grads)
        return dx.to(x.dtype), dw.to(weights.dtype), None, None, None, None


def fused_ep_moe(layer: "FusedEPMoE", x, weights, idx, params, grads):
    """Differentiable routed-expert sum. x (tokens, D) bf16; weights (tokens, k) fp32 (may require grad);
    ``params`` / ``grads``: this rank's stacked expert weights (bf16) and their fp32 gradient buffers."""
    return _FusedEPMoEFn.apply(x, weights, idx, layer, params, grads)


class EPMoERuntime:
    """What the model code calls for the routed experts of an expert-parallel layer: the fused kernels
    of one ``FusedEPMoE`` buffer set shared by all layers of the same shape, or of several sets used in
    rotation (pass a list): the backward of a layer reuses what its forward launch left in its set, so with as
    many sets as the model has MoE layers no forward launch has to be repeated in the backward pass; with fewer
    the layers whose set was reused recompute theirs. With gradient buffers in the layer's parameter dict
    (``<name>@grad``) and autograd on, the call is differentiable."""

    def __init__(self, layer):
        self.layers = list(layer) if isinstance(layer, (list, tuple)) else [layer]
        self.layer = self.layers[0]
        self._next = 0

    def __call__(self, x, weights, idx, params, grads=None):
        if grads is None:
            grads = {n: params.get(n + "@grad") for n in ("gate_proj", "up_proj", "down_proj")}
        train = torch.is_grad_enabled() and grads.get("gate_proj") is not None and self.layer.training
        if train:
            layer = self.layers[self._next % len(self.layers)]
            self._next += 1
            return fused_ep_moe(layer, x, weights, idx, params, grads)
        return self.layer.forward(x, weights, idx, params).to(x.dtype)

    def forward(self, x, weights, idx, params):
        return self(x, weights, idx, params)


class EPMoEInferenceRuntime:
    """Expert-parallel dispatcher for inference: one fused-kernel buffer set per token count (a prefill
    shape and a decode shape), bf16 or FP8. With ``fp8`` the layer's parameter dict must hold the
    pre-quantised weights of ``quantize_expert_weights_fp8`` (``gate_q`` ... ``sfb2``)."""

    def __init__(self, comm: Communicator, d_model: int, inter: int, n_experts: int, top_k: int, fp8: bool = False,
                 cap_factor: Optional[float] = None):
        self.comm, self.shape, self.fp8, self.cap_factor = comm, (d_model, inter, n_experts, top_k), fp8, cap_factor
        self._layers = {}

    def _layer(self, tokens: int):
        if tokens not in self._layers:
            cls = FusedEPMoEFp8 if self.fp8 else FusedEPMoE
            self._layers[tokens] = cls(self.comm, tokens, *self.shape, cap_factor=self.cap_factor)
        return self._layers[tokens]

    def forward(self, x, weights, idx, params, grads=None):
        """``grads`` is accepted (and ignored) so that the object also fits the callable form
        ``group(x, weights, idx, params, grads)`` of models/qwen35/moe.py:moe_layer."""
        return self._layer(x.shape[0]).forward(x.contiguous(), weights, idx, params).to(x.dtype)

    __call__ = forward


def quantize_stacked_experts_fp8(moe_params: dict) -> dict:
    """``moe_params``: a MoE parameter dict whose expert weights carry a leading layer axis
    ((L, E, D, I) / (L, E, I, D)). Returns a copy in which they are replaced by the stacked FP8 tensors
    (``gate_q`` ... ``sfb2`` with the same leading axis); the other entries are kept."""
    L = moe_params["gate_proj"].shape[0]
    per = [quantize_expert_weights_fp8({n: moe_params[n][l] for n in ("gate_proj", "up_proj", "down_proj")})
           for l in range(L)]
    out = {k: v for k, v in moe_params.items() if k not in ("gate_proj", "up_proj", "down_proj")}
    for k in ("gate_q", "up_q", "down_q", "sfb1", "sfb2"):
        out[k] = torch.stack([p[k] for p in per])
    return out


def shard_experts(params: dict, rank: int, world: int, names=("gate_proj", "up_proj", "down_proj"), _path=()) -> dict:
    """Copy of a parameter tree in which the stacked routed-expert weights (expert axis third from last)
    keep only the experts ``[rank * E / world, (rank + 1) * E / world)`` of this rank."""
    out = {}
    for k, v in params.items():
        if isinstance(v, dict):
            out[k] = shard_experts(v, rank, world, names, _path + (k,))
        elif k in names and v.dim() >= 3 and "mlp" not in _path:
            E = v.shape[-3]
            assert E % world == 0
            el = E // world
            out[k] = v.narrow(v.dim() - 3, rank * el, el).contiguous()
        else:
            out[k] = v
    return out


def is_expert_leaf(path, t, names=("gate_proj", "up_proj", "down_proj")) -> bool:
    """Predicate for ``TreeTrainEngine(local=...)``: the stacked routed-expert weights."""
    return path[-1] in names and t.dim() >= 3 and "shared" not in path[-1] and "mlp" not in path


def forward_tile_order(rows, n1: int, n2: int, grid: int):
    """Host model of the static tile order of the fused forward kernels (csrc/moe_common.cuh: build_tables /
    decode_tile), for tests and diagnostics. ``rows[e]``: rows received by local expert e; ``n1`` / ``n2``: column
    tiles of the gate|up and of the down GEMM; ``grid``: CTAs of the launch. Returns ``(lag, tiles)`` with
    ``tiles[t] = (expert, phase, m_tile, n_tile)``: the order is cut into ``E + lag`` slots, slot s holding the
    GEMM1 tiles of expert s followed by the GEMM2 tiles of expert s - lag, and the lag spans about two rounds of
    the grid at the average number of tiles per expert."""
    E = len(rows)
    mt = [(r + 127) // 128 for r in rows]
    total = sum(m * (n1 + n2) for m in mt)
    lag = (2 * grid * E + max(total, 1) - 1) // max(total, 1)
    lag = max(1, min(E, lag))
    tiles = []
    for s in range(E + lag):
        if s < E:
            tiles += [(s, 0, r % mt[s], r // mt[s]) for r in range(mt[s] * n1)]
        if s >= lag:
            e = s - lag
            tiles += [(e, 1, r % mt[e], r // mt[e]) for r in range(mt[e] * n2)]
    return lag, tiles


class NcclEPMoE:
    """Baseline: NCCL all-to-all dispatch and combine around per-expert GEMMs."""

    def __init__(self, group, n_experts: int):
        self.group, self.E = group, n_experts

    def forward(self, x, weights, idx, params):
        from ..models.qwen35.moe import expert_forward_ep
        return expert_forward_ep(x, weights, idx, params, self.group, self.E)
