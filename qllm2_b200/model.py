"""Drop-in PyTorch modules around the CUDA hot path: same class names, constructor arguments,
parameter names/shapes and call signatures as the reference's v11/model.py and v11/complex_ops.py,
so reference checkpoints (`state_dict`s) load unchanged.

Only the configuration the reference trains and ships is covered: head-scalar decay, additive
write, K >= 1 states (`n_states`), RoPE, GSP protect gate, ModSwish / ModReLU CGU.  The PAM scan,
the recurrent step and the tied head + cross-entropy run in libqllm2_pam_b200.so (no PyTorch
fallback); projections, norms and the gated unit are ordinary torch modules (cuBLAS GEMMs).

Reference map (file:line in the reference project):
  V11Config            v11/model.py:45-97          ComplexLinear      v11/complex_ops.py:146-172
  V11PAMLayer          v11/model.py:102-965        ComplexNorm        v11/complex_ops.py:175-189
  V11Block             v11/model.py:1021-1049      ComplexGatedUnit   v11/complex_ops.py:200-220
  V11LM                v11/model.py:1054-1260      ComplexEmbed       v11/complex_ops.py:223-235
  PRESETS / get_config v11/model.py:1265-1344      build_rope_cache   v11/complex_ops.py:261-266
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from . import fused_elementwise as FE
from . import ops
from .fused_ce import fused_linear_cross_entropy


# ------------------------------------------------------------------------------------ config
@dataclass
class V11Config:
    vocab_size: int = 50257
    dim: int = 384
    n_heads: int = 6
    head_dim: int = 64
    n_layers: int = 16
    expand: int = 3
    dropout: float = 0.1
    max_seq_len: int = 2048
    use_learned_pos: bool = False
    use_rope: bool = True
    use_gsp: bool = True
    fused_qkv: bool = True
    qk_norm: bool = False
    tie_weights: bool = True
    gradient_checkpointing: bool = True
    activation: str = "swish"
    chunk_size: int = 256
    decay_mode: str = "head"
    write_mode: str = "additive"
    n_states: int = 1
    delta_chunk: int = 64
    state_dt_spread: float = 2.0
    base_dt_bias: float = -4.0
    gate_content_aware: bool = False
    protect_gate_bias: float = -3.0
    routing_content_aware: bool = False
    state_compete: bool = False
    phase_init: str = "zero"
    route_balance_lambda: float = 0.0
    aux_loss_weight: float = 1.0
    fused_e3: bool = True
    recompute_pam_chunks: bool = False
    gamma_floor: float = 0.0
    gate_surprisal_lambda: float = 0.0
    gate_surprisal_tau: float = 1.0
    gate_surprisal_sign: float = 1.0


# ------------------------------------------------------------------------------------ complex helpers
def _magnitude(z: torch.Tensor) -> torch.Tensor:
    return torch.sqrt(z[..., 0] ** 2 + z[..., 1] ** 2 + 1e-8)


def _concat_planes(z: torch.Tensor) -> torch.Tensor:
    return torch.cat([z[..., 0], z[..., 1]], dim=-1)


def _complex_mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    ar, ai, br, bi = a[..., 0], a[..., 1], b[..., 0], b[..., 1]
    return torch.stack([ar * br - ai * bi, ar * bi + ai * br], dim=-1)


def build_rope_cache(max_len: int, head_dim: int) -> torch.Tensor:
    """[max_len, head_dim, 2]: (cos, sin) of position * 10000^(-j/head_dim), one band per channel."""
    inv = 1.0 / (10000.0 ** (torch.arange(head_dim).float() / head_dim))
    ang = torch.arange(max_len).float()[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1)


class ComplexLinear(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, bias: bool = True):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        gain = (2 / (in_dim + out_dim)) ** 0.5
        self.weight_real = nn.Parameter(torch.empty(out_dim, in_dim))
        self.weight_imag = nn.Parameter(torch.empty(out_dim, in_dim))
        nn.init.orthogonal_(self.weight_real, gain=gain)
        nn.init.orthogonal_(self.weight_imag, gain=gain)
        if bias:
            self.bias_real = nn.Parameter(torch.zeros(out_dim))
            self.bias_imag = nn.Parameter(torch.zeros(out_dim))
        else:
            self.register_parameter("bias_real", None)
            self.register_parameter("bias_imag", None)

    def block_weight(self) -> torch.Tensor:
        """[2*out, 2*in] real matrix acting on interleaved (re, im) columns: rows (o, re) = (Wr, -Wi),
        rows (o, im) = (Wi, Wr).  With it the complex product is ONE GEMM whose output is already
        interleaved.  Cached while no gradient is needed and the parameters are unchanged."""
        wr, wi = self.weight_real, self.weight_imag
        live = torch.is_grad_enabled() and (wr.requires_grad or wi.requires_grad)
        out_dtype = wr.dtype
        if wr.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16:
            out_dtype = torch.bfloat16          # written in the GEMM's dtype: no separate cast of the weight
        key = (wr._version, wi._version, wr.data_ptr(), wi.data_ptr(), wr.dtype, out_dtype)
        if not live and getattr(self, "_bw_key", None) == key:
            return self._bw
        if wr.is_cuda and wr.dtype in (torch.float32, torch.bfloat16):
            w = FE.block_weight(wr, wi, out_dtype)
        else:
            w = torch.stack([torch.stack([wr, -wi], dim=-1), torch.stack([wi, wr], dim=-1)], dim=1)
            w = w.view(2 * self.out_dim, 2 * self.in_dim)
        if not live:
            self._bw, self._bw_key = w.detach(), key
        return w

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-2]
        bias = None
        if self.bias_real is not None:
            bias = torch.stack([self.bias_real, self.bias_imag], dim=-1).view(-1)
        y = F.linear(x.reshape(*lead, 2 * self.in_dim), self.block_weight(), bias)
        return y.view(*lead, self.out_dim, 2)


class ComplexNorm(nn.Module):
    """RMS-normalise magnitudes, keep phases (v11/triton_kernels.py:489-494 is the arithmetic)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return FE.fused_complex_norm(z, self.scale, self.eps)      # CUDA only: the kernel wrapper refuses CPU tensors


class ModSwish(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.bias = nn.Parameter(torch.zeros(dim))
        self.beta = nn.Parameter(torch.ones(dim))

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return FE.fused_mod_swish(z, self.bias, self.beta)


class ModReLU(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.bias = nn.Parameter(torch.full((dim,), -0.1))

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return FE.fused_mod_relu(z, self.bias)


class ComplexGatedUnit(nn.Module):
    def __init__(self, dim: int, expand: int = 3, activation: str = "modrelu"):
        super().__init__()
        hidden = dim * expand
        self.gate_proj = ComplexLinear(dim, hidden, bias=False)
        self.up_proj = ComplexLinear(dim, hidden, bias=False)
        self.down_proj = ComplexLinear(hidden, dim, bias=False)
        if activation == "swish":
            self.act = ModSwish(hidden)
        elif activation == "modrelu":
            self.act = ModReLU(hidden)
        else:
            raise ValueError(f"activation '{activation}' is not supported by this package")

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        gate = self.gate_proj(z)
        up = self.act(self.up_proj(z))
        return self.down_proj(FE.fused_cgu_gate(gate, up))


class ComplexEmbed(nn.Module):
    def __init__(self, vocab_size: int, dim: int):
        super().__init__()
        self.dim = dim
        self.embed_real = nn.Embedding(vocab_size, dim)
        self.embed_imag = nn.Embedding(vocab_size, dim)
        nn.init.normal_(self.embed_real.weight, std=0.02)
        nn.init.normal_(self.embed_imag.weight, std=0.02)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return torch.stack([self.embed_real(ids), self.embed_imag(ids)], dim=-1)


def _dropout_mask(drop: nn.Dropout, like: torch.Tensor) -> torch.Tensor:
    return drop(torch.ones(like.shape[:-1], device=like.device, dtype=like.dtype)).unsqueeze(-1)


# ------------------------------------------------------------------------------------ PAM layer
class V11PAMLayer(nn.Module):
    """Matrix-state memory  S_t = gamma_t S_{t-1} + V_t (x) K_t^*,  Y_t = sum_k c_k S^k_t Q_t.

    forward(x [B,T,D,2], state=None, step_offset=0) -> (out [B,T,D,2], new_state) with new_state
    [B,H,d,d,2] (n_states == 1) or [K,B,H,d,d,2], exactly as the reference layer.
    """

    def __init__(self, cfg: V11Config, layer_idx: int = 0):
        super().__init__()
        if cfg.decay_mode != "head" or cfg.write_mode != "additive":
            raise ValueError("only decay_mode='head' with write_mode='additive' is implemented (the shipped configuration)")
        self.num_heads, self.head_dim = cfg.n_heads, cfg.head_dim
        inner = cfg.n_heads * cfg.head_dim
        self.inner_dim, self.dim = inner, cfg.dim
        self.fused_qkv, self.use_rope, self.use_gsp, self.qk_norm = cfg.fused_qkv, cfg.use_rope, cfg.use_gsp, cfg.qk_norm
        self.decay_mode, self.write_mode, self.n_states = cfg.decay_mode, cfg.write_mode, cfg.n_states
        self.chunk_size = cfg.chunk_size
        if cfg.fused_qkv:
            self.qkv_proj = ComplexLinear(cfg.dim, 3 * inner, bias=False)
        else:
            self.q_proj = ComplexLinear(cfg.dim, inner, bias=False)
            self.k_proj = ComplexLinear(cfg.dim, inner, bias=False)
            self.v_proj = ComplexLinear(cfg.dim, inner, bias=False)
        self.o_proj = ComplexLinear(inner, cfg.dim, bias=False)
        self.dt_proj = nn.Linear(cfg.dim * 2, cfg.n_heads)
        self.dt_bias = nn.Parameter(torch.zeros(cfg.n_heads) + cfg.base_dt_bias)
        self.gate_content_aware = cfg.gate_content_aware
        self.protect_gate_bias = cfg.protect_gate_bias
        self.routing_content_aware = cfg.routing_content_aware
        self.state_compete = cfg.state_compete
        self.phase_init = cfg.phase_init
        self.route_balance_lambda = cfg.route_balance_lambda
        self.gamma_floor = cfg.gamma_floor
        self.gate_surprisal_lambda = cfg.gate_surprisal_lambda
        if cfg.use_gsp:
            self.protect_gate = nn.Linear(cfg.dim * 2 if cfg.gate_content_aware else cfg.dim, cfg.n_heads)
            nn.init.constant_(self.protect_gate.bias, cfg.protect_gate_bias)
        if cfg.n_states > 1:
            self.state_dt_offset = nn.Parameter(torch.linspace(-cfg.state_dt_spread, cfg.state_dt_spread, cfg.n_states))
            route_in = cfg.dim * 2 if cfg.routing_content_aware else cfg.dim
            self.phase_proj = nn.Linear(route_in, cfg.n_heads * cfg.n_states)
            if cfg.state_compete:
                self.score_proj = nn.Linear(route_in, cfg.n_heads * cfg.n_states)
                nn.init.zeros_(self.score_proj.weight)
                nn.init.zeros_(self.score_proj.bias)
            self._init_phase_proj()
        if cfg.use_rope:
            self.register_buffer("rope_cache", build_rope_cache(cfg.max_seq_len, cfg.head_dim), persistent=False)
        self.dropout = nn.Dropout(cfg.dropout)
        self._route_aux = None
        self._gate_prob_bt = None

    def _init_phase_proj(self):
        if self.n_states <= 1:
            return
        K, H = self.n_states, self.num_heads
        if self.phase_init == "ortho":
            nn.init.orthogonal_(self.phase_proj.weight)
            nn.init.zeros_(self.phase_proj.bias)
            return
        nn.init.zeros_(self.phase_proj.weight)
        nn.init.zeros_(self.phase_proj.bias)
        if self.phase_init == "spread":
            per_state = [0.0, 2 * math.pi / 3, -2 * math.pi / 3] if K == 3 else [s * 2 * math.pi / K for s in range(K)]
            with torch.no_grad():
                self.phase_proj.bias.copy_(torch.tensor(per_state).repeat(H))

    # -- projections -------------------------------------------------------------------
    def _project(self, x: torch.Tensor, step_offset: int):
        B, T = x.shape[0], x.shape[1]
        H, d = self.num_heads, self.head_dim
        if self.fused_qkv:
            qkv = self.qkv_proj(x).view(B, T, 3, H, d, 2)
            q, k, v = (qkv[:, :, i].transpose(1, 2).contiguous() for i in range(3))
        else:
            q, k, v = (proj(x).view(B, T, H, d, 2).transpose(1, 2).contiguous()
                       for proj in (self.q_proj, self.k_proj, self.v_proj))
        if self.use_rope:
            end = step_offset + T
            if end > self.rope_cache.shape[0]:
                self.register_buffer("rope_cache", build_rope_cache(end * 2, d).to(x.device), persistent=False)
            rot = self.rope_cache[step_offset:end].to(dtype=x.dtype)
            q, k = _complex_mul(q, rot), _complex_mul(k, rot)
        if self.qk_norm:
            q, k = q / _magnitude(q).unsqueeze(-1), k / _magnitude(k).unsqueeze(-1)
        return q, k, v

    def _routing_input(self, x):
        return _concat_planes(x) if self.routing_content_aware else _magnitude(x)

    def _phase_and_alpha(self, x: torch.Tensor):
        B, T = x.shape[0], x.shape[1]
        H, K = self.num_heads, self.n_states
        r = self._routing_input(x)
        phase = self.phase_proj(r).view(B, T, H, K)
        if self.state_compete:
            weights = F.softmax(self.score_proj(r).view(B, T, H, K), dim=-1) * K
        else:
            weights = torch.ones(B, T, H, K, device=x.device, dtype=x.dtype)
        return phase, weights

    def _route_balance_loss(self, weights):
        if self.route_balance_lambda <= 0 or not self.state_compete or not self.training:
            return None
        mean_p = (weights / self.n_states).mean(dim=(0, 1))
        ent = -(mean_p * (mean_p + 1e-8).log()).sum(dim=-1)
        return -self.route_balance_lambda * ent.mean()

    def _gates(self, x: torch.Tensor):
        """gamma [K,B,H,T] for every state and omp = 1 - p [B,T,H] (None without the protect gate)
        (v11/model.py:630-655)."""
        K = self.n_states
        flat = _concat_planes(x)
        dt = self.dt_proj(flat) + self.dt_bias                                    # [B,T,H]
        if K > 1:
            dt = dt.unsqueeze(0) + self.state_dt_offset.view(K, 1, 1, 1)
        else:
            dt = dt.unsqueeze(0)
        base = torch.exp(-F.softplus(dt)).permute(0, 1, 3, 2)                    # [K,B,H,T]
        if self.gamma_floor and self.gamma_floor > 0.0:
            base = self.gamma_floor + (1.0 - self.gamma_floor) * base
        if not self.use_gsp:
            return base.contiguous(), None
        gate_in = flat if self.gate_content_aware else _magnitude(x)
        p_bth = torch.sigmoid(self.protect_gate(gate_in))                         # [B,T,H]
        protect = p_bth.transpose(1, 2)                                           # [B,H,T]
        if self.gate_surprisal_lambda > 0 and self.training:
            self._gate_prob_bt = protect.mean(dim=1)
        gamma = base * (1 - protect) + protect
        return gamma.contiguous(), 1 - p_bth

    def _fused_gates_ok(self, x: torch.Tensor) -> bool:
        """One kernel for the decay / protect / routing arithmetic unless a training-time auxiliary loss needs
        the intermediate tensors."""
        aux = self.training and ((self.route_balance_lambda > 0 and self.state_compete) or self.gate_surprisal_lambda > 0)
        return x.is_cuda and not aux and 1 <= self.n_states <= 4

    def gates_and_coef(self, x: torch.Tensor):
        """gamma [K,B,H,T], omp [B,T,H] or None, coef [K,B,H,T,2] or None for one layer input x [B,T,D,2]."""
        if not self._fused_gates_ok(x):
            gamma, omp = self._gates(x)
            return gamma, omp, self._coef(x)
        B, T = x.shape[0], x.shape[1]
        H, K, D = self.num_heads, self.n_states, self.dim
        x = x.contiguous()
        flat = x.view(B, T, 2 * D)                        # interleaved (re, im) columns: no copy

        def planar(lin):      # a Linear over [x_re | x_im] applied to the interleaved columns (weight columns permuted)
            w = lin.weight
            return F.linear(flat, w.view(w.shape[0], 2, D).transpose(1, 2).reshape(w.shape[0], 2 * D), lin.bias)

        fused_mag = x.dtype in (torch.float32, torch.bfloat16) and (x.numel() // 2) % 4 == 0
        mag = None
        pg = phase = score = None
        if self.use_gsp and self.gate_content_aware:
            # dt_proj and protect_gate read the same rows: one product with the two weight matrices stacked (a Linear
            # with a handful of outputs costs one pass over its input, forward and backward, whatever its width)
            lins = (self.dt_proj, self.protect_gate)
            w = torch.cat([l.weight.view(l.weight.shape[0], 2, D).transpose(1, 2).reshape(l.weight.shape[0], 2 * D) for l in lins])
            both = F.linear(flat, w, torch.cat([l.bias for l in lins]))
            dt, pg = both[..., :H], both[..., H:]
        else:
            dt = planar(self.dt_proj)
            if self.use_gsp:
                mag = FE.complex_magnitude(x) if fused_mag else _magnitude(x)
                pg = self.protect_gate(mag)
        if K > 1:
            if not self.routing_content_aware and mag is None:
                mag = FE.complex_magnitude(x) if fused_mag else _magnitude(x)
            proj = planar if self.routing_content_aware else (lambda lin: lin(mag))
            phase = proj(self.phase_proj).view(B, T, H, K)
            if self.state_compete:
                score = proj(self.score_proj).view(B, T, H, K)
        self._route_aux = None
        return FE.pam_gates(dt, pg, phase, score, self.dt_bias, self.state_dt_offset if K > 1 else None,
                            float(self.gamma_floor or 0.0), K)

    def _gamma_all_and_vprime(self, x: torch.Tensor, values: torch.Tensor):
        """gamma [K,B,H,T] and the protected value v' = (1 - p) v for values [B,H,T,d,2]."""
        gamma, omp = self._gates(x)
        if omp is None:
            return gamma, values
        return gamma, values * omp.transpose(1, 2)[..., None, None]

    def _fused_prep_ok(self, x: torch.Tensor) -> bool:
        d = self.head_dim
        return x.is_cuda and self.fused_qkv and not self.qk_norm and 4 <= d <= 128 and d & (d - 1) == 0

    def project_gated(self, x: torch.Tensor, step_offset: int = 0, positions: Optional[torch.Tensor] = None):
        """q, k, v' [B,H,T,d,2], gamma [K,B,H,T] and the read-out weights coef [K,B,H,T,2] (None when K == 1) of
        one layer input x [B,T,D,2].  `positions` [B,T]
        gives every token its own rotary position (continuous batching); otherwise step_offset + t."""
        if not self._fused_prep_ok(x):
            if positions is not None:
                raise ValueError("per-token positions need the fused projection path (fused_qkv, no qk_norm, CUDA)")
            q, k, v = self._project(x, step_offset)
            gamma, vprime = self._gamma_all_and_vprime(x, v)
            return q, k, vprime, gamma, self._coef(x)
        gamma, omp, coef = self.gates_and_coef(x)
        rope = None
        if self.use_rope:
            if positions is None and step_offset + x.shape[1] > self.rope_cache.shape[0]:
                self.register_buffer("rope_cache", build_rope_cache((step_offset + x.shape[1]) * 2, self.head_dim).to(x.device),
                                     persistent=False)
            rope = self.rope_cache
        q, k, vprime = FE.pam_prep(self.qkv_proj(x), rope, omp, n_heads=self.num_heads, head_dim=self.head_dim,
                                   positions=positions, offset=step_offset)
        return q, k, vprime, gamma, coef

    def _gamma_and_vprime(self, x, values, state_offset: float = 0.0):
        """Single-state form kept for callers of the reference API (v11/model.py:308-350)."""
        flat = _concat_planes(x)
        base = torch.exp(-F.softplus(self.dt_proj(flat) + self.dt_bias + state_offset)).transpose(1, 2)
        if self.gamma_floor and self.gamma_floor > 0.0:
            base = self.gamma_floor + (1.0 - self.gamma_floor) * base
        if not self.use_gsp:
            return base.contiguous(), values
        gate_in = flat if self.gate_content_aware else _magnitude(x)
        protect = torch.sigmoid(self.protect_gate(gate_in)).transpose(1, 2)
        return (base * (1 - protect) + protect).contiguous(), values * (1 - protect)[..., None, None]

    def _coef(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Read-out weights c_k = alpha_k e^{i phi_k} as [K,B,H,T,2]; None when K == 1."""
        if self.n_states == 1:
            return None
        phase, weights = self._phase_and_alpha(x)
        self._route_aux = self._route_balance_loss(weights)
        phase, weights = phase.permute(3, 0, 2, 1), weights.permute(3, 0, 2, 1)
        return torch.stack([weights * torch.cos(phase), weights * torch.sin(phase)], dim=-1).contiguous()

    # -- reference-named scan entry points ------------------------------------------------
    def _forward_chunked_head(self, queries, keys, protected_values, decay_gamma, head_dim):
        y, s = ops.pam_scan(queries, keys, protected_values, decay_gamma, head_dim=head_dim, chunk=self.chunk_size)
        return y, s[0].to(queries.dtype)

    def _recur_step_additive(self, memory_state, decay_gamma, value_t, key_t, query_t):
        """One step on a [B,H,d,d,2] state; returns (y [B,H,d,2], new state) without touching the input."""
        B = memory_state.shape[0]
        pool = memory_state.detach().clone().contiguous().unsqueeze(1).unsqueeze(1)   # [B,1,1,H,d,d,2]
        slots = torch.arange(B, dtype=torch.int32, device=memory_state.device)
        y = ops.pam_decode_step(pool, slots, query_t, key_t, value_t, decay_gamma)
        return y, pool[:, 0, 0]

    # -- forward ---------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, state=None, step_offset: int = 0):
        B, T = x.shape[0], x.shape[1]
        H, d, K = self.num_heads, self.head_dim, self.n_states
        q, k, vprime, gamma, coef = self.project_gated(x, step_offset)
        if state is None and T > 1:
            y, s = ops.pam_scan(q, k, vprime, gamma, coef=coef, head_dim=d, chunk=self.chunk_size, token_major=True)
            new_state = (s[0] if K == 1 else s).to(x.dtype)
        else:
            y, new_state = self._recurrent(q, k, vprime, gamma, coef, state)
            y = y.transpose(1, 2).contiguous().view(B, T, self.inner_dim, 2)
        out = self.o_proj(y)
        if self.training and self.dropout.p > 0:
            out = out * _dropout_mask(self.dropout, out)
        return out, new_state

    @torch.no_grad()
    def _recurrent(self, q, k, vprime, gamma, coef, state):
        """Token loop on the O(1) step kernel (v11/model.py:845-925)."""
        B, H, T, d = q.shape[:4]
        K = self.n_states
        if state is None:
            pool = torch.zeros(B, 1, K, H, d, d, 2, device=q.device, dtype=q.dtype)
        elif K == 1:
            pool = state.detach().clone().view(B, 1, 1, H, d, d, 2)
        else:
            pool = state.detach().permute(1, 0, 2, 3, 4, 5).contiguous().view(B, 1, K, H, d, d, 2)
        slots = torch.arange(B, dtype=torch.int32, device=q.device)
        qs = q * (d ** -0.5)
        ys = []
        for t in range(T):
            c_t = None if coef is None else coef[:, :, :, t].contiguous()
            ys.append(ops.pam_decode_step(pool, slots, qs[:, :, t].contiguous(), k[:, :, t].contiguous(),
                                          vprime[:, :, t].contiguous(), gamma[:, :, :, t].contiguous(), c_t))
        y = torch.stack(ys, dim=2)
        new_state = pool[:, 0, 0] if K == 1 else pool[:, 0].permute(1, 0, 2, 3, 4, 5).contiguous()
        return y, new_state


# ------------------------------------------------------------------------------------ block / LM
class V11Block(nn.Module):
    """Pre-norm residual block: channel mix (CGU) then sequence mix (PAM)."""

    def __init__(self, cfg: V11Config, layer_idx: int = 0):
        super().__init__()
        self.norm1 = ComplexNorm(cfg.dim)
        self.cgu = ComplexGatedUnit(cfg.dim, cfg.expand, activation=cfg.activation)
        self.cgu_scale = nn.Parameter(torch.tensor(1.0))
        self.cgu_dropout = nn.Dropout(cfg.dropout)
        self.norm2 = ComplexNorm(cfg.dim)
        self.pam = V11PAMLayer(cfg, layer_idx=layer_idx)
        self.pam_scale = nn.Parameter(torch.tensor(0.1))

    def forward(self, x, pam_state=None, step_offset: int = 0):
        mixed = self.cgu(self.norm1(x))
        if self.training and self.cgu_dropout.p > 0:
            mixed = mixed * _dropout_mask(self.cgu_dropout, mixed)
        x = self._residual(x, mixed, self.cgu_scale)
        pam_out, new_state = self.pam(self.norm2(x), state=pam_state, step_offset=step_offset)
        return self._residual(x, pam_out, self.pam_scale), new_state

    @staticmethod
    def _residual(x, delta, scale):
        if not x.is_cuda:
            raise _lib.QPamError("V11Block runs on CUDA tensors only (there is no CPU path in this package)")
        if x.numel() % 4 == 0 and x.dtype in (torch.float32, torch.bfloat16) and delta.dtype in (torch.float32, torch.bfloat16):
            return FE.scaled_residual(x, delta, scale)
        return x + delta * scale        # other dtypes (fp16, fp64): the residual add stays a torch operator


class ComplexPosEmbed(nn.Module):
    def __init__(self, max_seq_len: int, dim: int):
        super().__init__()
        self.max_seq_len = max_seq_len
        self.pos_embed = nn.Embedding(max_seq_len, dim)
        nn.init.normal_(self.pos_embed.weight, std=0.02)

    def forward(self, z, step_offset: int = 0):
        end = step_offset + z.shape[1]
        if end > self.max_seq_len:
            raise ValueError(f"Position range [{step_offset}, {end}) exceeds max_seq_len {self.max_seq_len}")
        pos = self.pos_embed(torch.arange(step_offset, end, device=z.device))
        return z + pos[None, :, :, None]


class V11LM(nn.Module):
    """ComplexEmbed -> V11Block x n_layers -> tied complex LM head."""

    def __init__(self, cfg: V11Config):
        super().__init__()
        self.config = cfg
        self.embed = ComplexEmbed(cfg.vocab_size, cfg.dim)
        self.pos_embed = ComplexPosEmbed(cfg.max_seq_len, cfg.dim) if cfg.use_learned_pos else None
        self.embed_norm = ComplexNorm(cfg.dim)
        self.blocks = nn.ModuleList([V11Block(cfg, layer_idx=i) for i in range(cfg.n_layers)])
        self.output_norm = ComplexNorm(cfg.dim)
        self.lm_head_proj = ComplexLinear(cfg.dim, cfg.dim)
        self.lm_head_norm = ComplexNorm(cfg.dim)
        self._init_weights()

    def _init_weights(self):
        tied = {self.embed.embed_real, self.embed.embed_imag}
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Embedding) and m not in tied:
                nn.init.normal_(m.weight, std=0.02)
        for m in self.modules():
            if isinstance(m, V11PAMLayer):
                if m.use_gsp:
                    nn.init.constant_(m.protect_gate.bias, m.protect_gate_bias)
                m._init_phase_proj()

    # -- stack -----------------------------------------------------------------------------
    def _embed(self, input_ids, step_offset):
        z = self.embed(input_ids)
        if self.pos_embed is not None:
            z = self.pos_embed(z, step_offset=step_offset)
        return self.embed_norm(z)

    def _aux(self, device):
        total = None
        for blk in self.blocks:
            a = getattr(blk.pam, "_route_aux", None)
            if a is not None:
                total = a if total is None else total + a
        return total if total is not None else torch.zeros((), device=device)

    def _run_blocks(self, z, states, step_offset, checkpoint):
        new_states = []
        for i, blk in enumerate(self.blocks):
            s = states[i] if states is not None else None
            if checkpoint:
                from torch.utils.checkpoint import checkpoint as ckpt
                z, ns = ckpt(lambda zz, b=blk: b(zz, pam_state=None, step_offset=step_offset), z, use_reentrant=False)
            else:
                z, ns = blk(z, pam_state=s, step_offset=step_offset)
            new_states.append(ns)
        return z, new_states

    def _head_hidden(self, z):
        return self.lm_head_norm(self.lm_head_proj(self.output_norm(z)))

    def forward(self, input_ids, states=None, step_offset: int = 0, labels=None):
        z = self._embed(input_ids, step_offset)
        ckpt = self.config.gradient_checkpointing and self.training and states is None
        z, new_states = self._run_blocks(z, states, step_offset, ckpt)
        lm = self._head_hidden(z)
        logits = lm[..., 0] @ self.embed.embed_real.weight.T + lm[..., 1] @ self.embed.embed_imag.weight.T
        return logits, new_states, self._aux(input_ids.device)

    def _hidden_to_lm(self, input_ids, step_offset: int = 0):
        z = self._embed(input_ids, step_offset)
        ckpt = self.config.gradient_checkpointing and self.training
        z, _ = self._run_blocks(z, None, step_offset, ckpt)
        lm = self._head_hidden(z)
        probs = [b.pam._gate_prob_bt for b in self.blocks if getattr(b.pam, "_gate_prob_bt", None) is not None]
        return lm, self._aux(input_ids.device), (torch.stack(probs, dim=0) if probs else None)

    def tied_head_matrices(self, lm):
        """H = [lm_r | lm_i] [N, 2D] and W = [E_r | E_i] [V, 2D] of the tied head."""
        H = torch.cat([lm[..., 0], lm[..., 1]], dim=-1).reshape(-1, 2 * lm.shape[-2])
        W = torch.cat([self.embed.embed_real.weight, self.embed.embed_imag.weight], dim=-1)
        return H, W

    def ce_from_lm(self, lm, labels, loss_mask=None, ignore_index=-100, chunk: int = 4096):
        H, W = self.tied_head_matrices(lm)
        if H.is_cuda and torch.is_autocast_enabled("cuda"):
            # the reference's head matmuls run in the autocast dtype; here that selects the tensor-core kernels
            H = H.to(torch.get_autocast_dtype("cuda"))
        if H.dtype != W.dtype:
            W = W.to(H.dtype)
        mask = loss_mask.reshape(-1) if loss_mask is not None else None
        return fused_linear_cross_entropy(H, W, labels.reshape(-1), mask=mask, chunk=chunk, ignore_index=ignore_index)

    def fused_ce_loss(self, input_ids, labels, loss_mask=None, ignore_index=-100, chunk: int = 4096):
        lm, aux, _ = self._hidden_to_lm(input_ids)
        return self.ce_from_lm(lm, labels, loss_mask=loss_mask, ignore_index=ignore_index, chunk=chunk), aux

    @torch.no_grad()
    def greedy_next(self, lm_last):
        """argmax of the tied head for hidden rows lm_last [B, D, 2] without forming logits."""
        H, W = self.tied_head_matrices(lm_last.unsqueeze(1))
        ids, _ = ops.head_argmax(H.contiguous(), W.to(H.dtype).contiguous())
        return ids

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=100, temperature=1.0, top_k=50, top_p=0.0,
                 repetition_penalty=1.0, eos_token_id=None, fused: bool = True):
        """Prefill once (parallel scan), then one O(1) recurrent step per token.  temperature <= 0
        selects greedy decoding (arg-max of the logits); otherwise the reference's sampling block
        (v11/model.py:1221-1244) runs as one kernel per token (`ops.sample_logits`).  The loop runs on the packed
        forward with the decode step replayed from a CUDA graph (`fused=False` keeps the module-by-module loop)."""
        self.eval()
        greedy = temperature is None or temperature <= 0

        def sample(nl, out):
            """nl: logits [B, V] of the last position; out: token ids so far [B, T] (for the repetition penalty)."""
            if greedy:
                return nl.argmax(dim=-1, keepdim=True)
            # temperature, penalty, top-k, top-p and the draw in one kernel (random numbers from torch's generator)
            return ops.sample_logits(nl, temperature=temperature, top_k=top_k, top_p=top_p,
                                     repetition_penalty=repetition_penalty,
                                     history=out.contiguous() if repetition_penalty != 1.0 else None)[:, None]

        if fused and input_ids.is_cuda and max_new_tokens > 0:
            from .fused_forward import FusedForward
            if FusedForward.unsupported_reason(self) is None:
                from .serving import generate_fused
                sample.greedy = greedy
                return generate_fused(self, input_ids, max_new_tokens, sample, eos_token_id=eos_token_id)
        out = input_ids.clone()
        logits, states, _ = self.forward(out)
        step = out.shape[1]
        done = torch.zeros(out.shape[0], dtype=torch.bool, device=out.device)
        for _ in range(max_new_tokens):
            nxt = sample(logits[:, -1].float(), out)
            out = torch.cat([out, nxt], dim=1)
            if eos_token_id is not None:
                done |= nxt.squeeze(1) == eos_token_id
                if bool(done.all()):
                    break
            logits, states, _ = self.forward(nxt, states=states, step_offset=step)
            step += 1
        return out

    def count_parameters(self) -> Dict[str, int]:
        n = lambda mods: sum(p.numel() for m in mods for p in m.parameters())
        embed = n([self.embed] + ([self.pos_embed] if self.pos_embed is not None else []))
        blocks, head = n(self.blocks), n([self.lm_head_proj, self.lm_head_norm])
        norms = n([self.embed_norm, self.output_norm])
        return {"embedding (tied)": embed, "blocks": blocks, "norms": norms, "lm_head": head,
                "total": embed + blocks + head + norms}


# ------------------------------------------------------------------------------------ presets
def _flat(**kw) -> V11Config:
    cfg = V11Config(vocab_size=50257, dim=384, n_heads=6, head_dim=64, n_layers=16, expand=3, dropout=0.1,
                    max_seq_len=2048, activation="swish", chunk_size=256)
    for key, val in kw.items():
        setattr(cfg, key, val)
    return cfg


_TINY = dict(vocab_size=50257, dim=64, n_heads=2, head_dim=32, n_layers=2, expand=2, dropout=0.0,
             max_seq_len=512, chunk_size=64, gradient_checkpointing=False)
_CHAT = dict(n_states=3, state_dt_spread=2.0, vocab_size=50261, gate_content_aware=True)

PRESETS = {
    "v11_baseline": _flat(),
    "v11_e3_multistate": _flat(n_states=2, state_dt_spread=2.0),
    "v11_e3_k3": _flat(n_states=3, state_dt_spread=2.0, gate_content_aware=True),
    "v11_e3_k3_chat": _flat(**_CHAT),
    "v11_e3_k3_chat_gate": _flat(**_CHAT),
    "v11_e3_k3_chat_recall": _flat(**_CHAT, gamma_floor=0.98, gate_surprisal_lambda=0.1, gate_surprisal_tau=1.0,
                                   gate_surprisal_sign=1.0),
    "v11_e3_k3_chat_compete": _flat(**_CHAT, routing_content_aware=True, state_compete=True, phase_init="spread",
                                    route_balance_lambda=0.01),
    "tiny": V11Config(**_TINY),
    "tiny_e3": V11Config(**_TINY, n_states=2),
}


def get_config(preset: str = "v11_baseline") -> V11Config:
    if preset not in PRESETS:
        raise ValueError(f"Unknown preset '{preset}'. Available: {list(PRESETS.keys())}")
    return copy.deepcopy(PRESETS[preset])
