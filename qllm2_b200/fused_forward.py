"""Inference-only forward of a V11LM through packed weights and the fused block kernels.

A V11 block at inference is four projections with element-wise work between them.  The module
path (`V11Block.forward`, mirroring v11/model.py) spends most of a decode step launching ~80 small
operators per layer; here a layer is

    GEMM gate|up -> k_act_gate_packed -> GEMM down -> k_residual_cnorm
    -> GEMM qkv|gates (-> GEMM gates on |x|) -> k_pam_front -> scan or decode step -> GEMM o
    -> k_residual_cnorm (which also produces the next layer's pre-norm)

with every weight packed once: complex projections as one real block matrix acting on interleaved
(re, im) columns, the small gate/routing Linears appended as extra output columns of the qkv
projection (their planar-input weights permuted to the interleaved column order).  The GEMMs are
library calls (cuBLAS through `F.linear`); everything between them is this package's kernels.
Weights are snapshots: build a new `FusedForward` after changing the model's parameters.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib, ops
from ._lib import check, dtype_code, ptr, stream_ptr
from .model import ModSwish, V11LM, build_rope_cache


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().float().contiguous()


class FusedForward:
    def __init__(self, model: V11LM, max_position: int = 8192):
        cfg = model.config
        why = self.unsupported_reason(model)
        if why:
            raise _lib.QPamError(f"FusedForward: {why}")
        p = next(model.parameters())
        self.model, self.cfg = model, cfg
        self.device, self.dtype = p.device, p.dtype
        self.D, self.H, self.d, self.K = cfg.dim, cfg.n_heads, cfg.head_dim, cfg.n_states
        self.inner = cfg.n_heads * cfg.head_dim
        self.rope = build_rope_cache(max_position, cfg.head_dim).to(self.device) if cfg.use_rope else None
        self.embed_scale = _f32(model.embed_norm.scale)
        self.out_scale = _f32(model.output_norm.scale)
        self.head_norm_scale = _f32(model.lm_head_norm.scale)
        hp = model.lm_head_proj
        self.w_head_proj = hp.block_weight().detach().to(self.dtype).contiguous()
        self.b_head_proj = (None if hp.bias_real is None else
                            torch.stack([hp.bias_real, hp.bias_imag], -1).reshape(-1).detach().to(self.dtype))
        self.w_vocab = torch.cat([model.embed.embed_real.weight, model.embed.embed_imag.weight], -1).detach().to(self.dtype).contiguous()
        self.layers = [self.pack_block(blk, self.dtype) for blk in model.blocks]

    @staticmethod
    def unsupported_reason(model: V11LM) -> Optional[str]:
        cfg = model.config
        d = cfg.head_dim
        if not cfg.fused_qkv or cfg.qk_norm:
            return "needs fused_qkv without qk_norm"
        if cfg.use_learned_pos:
            return "learned position embeddings are not packed"
        if d < 4 or d > 128 or d & (d - 1) or cfg.n_heads > 64:
            return "head_dim must be a power of two in [4,128] and n_heads <= 64"
        if cfg.dim % 4 or (cfg.dim * cfg.expand) % 4:
            return "dim and dim*expand must be multiples of 4"
        p = next(model.parameters())
        if not p.is_cuda or p.dtype not in (torch.float32, torch.bfloat16):
            return "needs a CUDA model in float32 or bfloat16"
        return None

    # ---------------------------------------------------------------------------------- packing
    @staticmethod
    def pack_block(blk, dtype) -> SimpleNamespace:
        """Packed weights of one V11Block (any device): `w_gu` [4*hidden, 2D] = gate | up block matrices,
        `w_down`, `w_front` = qkv block matrix followed by the gate / routing Linears that read the layer
        input (columns permuted from [re | im] planes to interleaved order; `cols[name]` = ("a", column)),
        `w_mag` = the Linears that read |x| (`cols[name]` = ("m", column)), `w_o`, and fp32 parameters."""
        cgu, pam = blk.cgu, blk.pam
        D, H, K, T = pam.dim, pam.num_heads, pam.n_states, dtype
        inner, device = pam.inner_dim, blk.norm1.scale.device
        L = SimpleNamespace()
        L.n1, L.n2 = _f32(blk.norm1.scale), _f32(blk.norm2.scale)
        L.hidden = cgu.gate_proj.out_dim
        L.w_gu = torch.cat([cgu.gate_proj.block_weight(), cgu.up_proj.block_weight()], 0).detach().to(T).contiguous()
        L.act_bias = _f32(cgu.act.bias)
        L.act_beta = _f32(cgu.act.beta) if isinstance(cgu.act, ModSwish) else None
        L.w_down = cgu.down_proj.block_weight().detach().to(T).contiguous()
        L.cgu_scale, L.pam_scale = _f32(blk.cgu_scale).view(1), _f32(blk.pam_scale).view(1)
        L.w_o = pam.o_proj.block_weight().detach().to(T).contiguous()
        L.dt_bias = _f32(pam.dt_bias)
        L.dt_off = _f32(pam.state_dt_offset) if K > 1 else None
        L.gamma_floor = float(pam.gamma_floor or 0.0)

        def interleaved_cols(lin):      # a Linear over [x_re | x_im] -> the same Linear over interleaved (re, im) columns
            w = lin.weight.detach()
            return w.view(w.shape[0], 2, D).transpose(1, 2).reshape(w.shape[0], 2 * D)

        rows_a, bias_a, rows_m, bias_m = [pam.qkv_proj.block_weight().detach()], [torch.zeros(6 * inner, device=device)], [], []
        L.cols = {}

        def add(name, lin, content_aware):
            if content_aware:
                L.cols[name] = ("a", sum(r.shape[0] for r in rows_a))
                rows_a.append(interleaved_cols(lin))
                bias_a.append(lin.bias.detach())
            else:
                L.cols[name] = ("m", sum(r.shape[0] for r in rows_m))
                rows_m.append(lin.weight.detach())
                bias_m.append(lin.bias.detach())

        add("dt", pam.dt_proj, True)
        if pam.use_gsp:
            add("pg", pam.protect_gate, pam.gate_content_aware)
        if K > 1:
            add("phase", pam.phase_proj, pam.routing_content_aware)
            if pam.state_compete:
                add("score", pam.score_proj, pam.routing_content_aware)
        n_a = sum(r.shape[0] for r in rows_a)
        pad = (-n_a) % 8            # rows of the projection output stay 16-byte aligned
        if pad:
            rows_a.append(torch.zeros(pad, 2 * D, device=device))
            bias_a.append(torch.zeros(pad, device=device))
        L.w_front = torch.cat([r.float() for r in rows_a], 0).to(T).contiguous()
        L.b_front = torch.cat([b.float() for b in bias_a], 0).to(T).contiguous()
        L.w_mag = torch.cat([r.float() for r in rows_m], 0).to(T).contiguous() if rows_m else None
        L.b_mag = torch.cat([b.float() for b in bias_m], 0).to(T).contiguous() if rows_m else None
        return L

    # ---------------------------------------------------------------------------------- kernels
    def _res_norm(self, z, delta, res_scale, norm_scale, want_mag=False):
        N = z.shape[0]
        xn = torch.empty_like(z)
        mag = torch.empty(N, self.D, dtype=z.dtype, device=z.device) if want_mag else None
        check(_lib.lib().qpam_residual_cnorm_fwd(ptr(z), ptr(delta), ptr(res_scale), ptr(norm_scale), ptr(xn), ptr(mag),
                                                 dtype_code(z.dtype), N, self.D, 1e-6, stream_ptr()), "qpam_residual_cnorm_fwd")
        return xn, mag

    def _front(self, L, raw, rawm, B, T, positions, offset, q_scale):
        H, d, K = self.H, self.d, self.K
        dev, dt = raw.device, raw.dtype
        q, k, v = (torch.empty(B, H, T, d, 2, dtype=dt, device=dev) for _ in range(3))
        gamma = torch.empty(K, B, H, T, dtype=torch.float32, device=dev)
        coef = torch.empty(K, B, H, T, 2, dtype=torch.float32, device=dev) if K > 1 else None
        a = _lib.FrontArgs()
        es = raw.element_size()

        def col(name):
            if name not in L.cols:
                return None, 0
            src, off = L.cols[name]
            base = raw if src == "a" else rawm
            return base.data_ptr() + off * es, base.shape[1]

        a.qkv, a.ld_qkv = raw.data_ptr(), raw.shape[1]
        a.dt, a.ld_dt = col("dt")
        a.pg, a.ld_pg = col("pg")
        a.phase, a.ld_phase = col("phase")
        a.score, a.ld_score = col("score")
        a.dt_bias, a.state_dt_offset = ptr(L.dt_bias), ptr(L.dt_off)
        a.rope, a.rope_len = ptr(self.rope), 0 if self.rope is None else self.rope.shape[0]
        a.positions, a.offset = ptr(positions), int(offset)
        a.q, a.k, a.v, a.gamma, a.coef = ptr(q), ptr(k), ptr(v), ptr(gamma), ptr(coef)
        a.gamma_floor, a.q_scale = L.gamma_floor, float(q_scale)
        a.B, a.T, a.H, a.d, a.K, a.io_dtype = B, T, H, d, K, dtype_code(dt)
        check(_lib.lib().qpam_pam_front_fwd(a, stream_ptr()), "qpam_pam_front_fwd")
        return q, k, v, gamma, coef

    # ---------------------------------------------------------------------------------- forward
    @torch.no_grad()
    def hidden(self, ids: torch.Tensor, mix, positions: Optional[torch.Tensor] = None, offset: int = 0):
        """Run the blocks over ids [B, T]; `mix(layer, q, k, v, gamma, coef) -> y [B*T, inner*2]` is the
        sequence-mixing step (a scan at prefill, the recurrent step at decode).  Returns the final
        residual stream normalised by output_norm, [B*T, D, 2]."""
        m, D = self.model, self.D
        B, T = ids.shape
        N = B * T
        if self.rope is not None and positions is None and offset + T > self.rope.shape[0]:
            raise _lib.QPamError("position beyond max_position of this FusedForward")
        if positions is not None:
            positions = positions.reshape(-1).to(torch.int64).contiguous()
        z = torch.stack([m.embed.embed_real(ids), m.embed.embed_imag(ids)], dim=-1).reshape(N, D, 2).to(self.dtype)
        z, _ = self._res_norm(z, None, None, self.embed_scale)          # embed_norm
        xn, _ = self._res_norm(z, None, None, self.layers[0].n1)
        lib = _lib.lib()
        for li, L in enumerate(self.layers):
            gu = F.linear(xn.view(N, 2 * D), L.w_gu)                      # [N, 4*hidden]
            gated = torch.empty(N, L.hidden, 2, dtype=z.dtype, device=z.device)
            check(lib.qpam_act_gate_packed_fwd(ptr(gu), gu.shape[1], dtype_code(gu.dtype), ptr(L.act_bias), ptr(L.act_beta),
                                               ptr(gated), N, L.hidden, stream_ptr()), "qpam_act_gate_packed_fwd")
            dn = F.linear(gated.view(N, 2 * L.hidden), L.w_down)
            xn2, mag = self._res_norm(z, dn, L.cgu_scale, L.n2, want_mag=L.w_mag is not None)
            raw = F.linear(xn2.view(N, 2 * D), L.w_front, L.b_front)
            rawm = F.linear(mag, L.w_mag, L.b_mag) if L.w_mag is not None else None
            q, k, v, gamma, coef = self._front(L, raw, rawm, B, T, positions, offset, mix.q_scale)
            y = mix(li, q, k, v, gamma, coef)                              # [N, inner*2]
            o = F.linear(y, L.w_o)
            nxt = self.layers[li + 1].n1 if li + 1 < len(self.layers) else self.out_scale
            xn, _ = self._res_norm(z, o, L.pam_scale, nxt)
        return xn                                                          # output_norm(z)

    @torch.no_grad()
    def head_hidden(self, xn: torch.Tensor) -> torch.Tensor:
        """lm_head_norm(lm_head_proj(.)) of rows [n, D, 2] already normalised by output_norm."""
        n = xn.shape[0]
        h = F.linear(xn.reshape(n, 2 * self.D), self.w_head_proj, self.b_head_proj).view(n, self.D, 2)
        h, _ = self._res_norm(h, None, None, self.head_norm_scale)
        return h

    @torch.no_grad()
    def logits(self, lm: torch.Tensor) -> torch.Tensor:
        """Tied-head logits [n, V] (float32) of rows lm [n, D, 2]: Re(lm . conj(E)) as one real GEMM
        (v11/model.py:1136-1139); only the sampling path needs them."""
        Hm = torch.cat([lm[..., 0], lm[..., 1]], dim=-1)
        if Hm.dtype == torch.bfloat16 and self.w_vocab.dtype == torch.bfloat16:
            return ops.head_logits(Hm, self.w_vocab).float()       # the cross-entropy's tensor-core GEMM, bf16 tiles out
        return F.linear(Hm, self.w_vocab).float()

    @torch.no_grad()
    def greedy_next(self, lm: torch.Tensor) -> torch.Tensor:
        """argmax over the tied head for rows lm [n, D, 2] (no logits are formed)."""
        Hm = torch.cat([lm[..., 0], lm[..., 1]], dim=-1).contiguous()
        ids, _ = ops.head_argmax(Hm, self.w_vocab)
        return ids
