"""Latent attention: keys and values of every head are products of one low-rank latent row per token,
and only that row is cached.

    c_q = norm(W_dq x)            q_h = W_uq,h c_q              (heads x dim)
    c   = norm(W_dkv x)           k_h = W_uk,h c,  v_h = W_uv,h c
    o_h = softmax(scale q_h K_h^T) V_h * sigmoid(w_g,h . x)     y = W_o [o_1 .. o_H]

Because k and v are linear in c, the products with W_uk and W_uv move to the query's and the output's side:

    q_h . k_h(j) = (W_uk,h^T q_h) . c(j)            sum_j p_j v_h(j) = W_uv,h (sum_j p_j c(j))

so the attention itself is multi-query attention with ONE shared "kv head" whose key and value are both the
latent row, of head size kv_rank, and it runs on the library's attention kernels as they are (tensor-core
prompt and decode kernels at kv_rank 64 / 128 / 256, the generic ones otherwise), with the window and the
scale as their parameters.  The per-head matrices are folded into their neighbours when the model is loaded,
in float64 and rounded once:  W_qk = [W_uk,h^T W_uq,h]_h  (heads*kv_rank x q_rank)  and
W_ov = [W_o,h W_uv,h]_h  (width x heads*kv_rank); the gate, a scalar per head, commutes with W_uv,h and
multiplies the attention's output.  The cache line keeps the latent only (one row per position, no value pool).
There are no positions in this mixer.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .attention import AttentionMixer
from .base import MIXERS, CacheNeed, HeadShape
from .linear import project, stack_rows
from .spec import PartSpec


@MIXERS.register("latent_attention")
class LatentAttentionMixer(AttentionMixer):
    def __init__(self, spec: PartSpec):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.q_rank = int(p["q_rank"])
        self.kv_rank = int(p["kv_rank"])
        self.eps = float(p["eps"])
        # the attention kernels take head sizes in whole 16-byte pieces: a latent of another size is carried with
        # zero columns behind it (they add nothing to a score and meet zero columns of the output matrix)
        self.rank_pad = (self.kv_rank + 7) // 8 * 8
        inner = PartSpec("attention", {
            "hidden_size": self.hidden, "n_heads": self.n_heads, "n_kv_heads": 1, "head_dim": self.rank_pad,
            "scale": float(p["scale"]), "softcap": None, "window": p.get("window"),
            "position": PartSpec("none", {"head_dim": self.rank_pad})})
        super().__init__(inner)
        self.spec = spec
        self.w_in: Optional[torch.Tensor] = None        # [q_rank + kv_rank, width]: W_dq over W_dkv
        self.w_gate: Optional[torch.Tensor] = None      # [heads, width]
        self.w_qk: Optional[torch.Tensor] = None        # [heads * kv_rank, q_rank]
        self.w_ov: Optional[torch.Tensor] = None        # [width, heads * kv_rank]
        self.norm_q: Optional[torch.Tensor] = None
        self.norm_kv: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"])
        rq, rkv = int(p["q_rank"]), int(p["kv_rank"])
        M, N = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_SCALE
        return {"dq": ((rq, W), M), "dq_norm": ((rq,), N), "uq": ((H * d, rq), M),
                "dkv": ((rkv, W), M), "dkv_norm": ((rkv,), N), "uk": ((H * d, rkv), M), "uv": ((H * vd, rkv), M),
                "gate": ((H, W), M), "o": ((W, H * vd), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        H, d, vd, r = self.n_heads, self.dim, self.vdim, self.kv_rank
        self.w_in = stack_rows([tensors["dq"], tensors["dkv"]])
        self.w_gate = tensors["gate"].contiguous()
        self.norm_q = tensors["dq_norm"].contiguous()
        self.norm_kv = tensors["dkv_norm"].contiguous()
        wide = torch.float64
        uq = tensors["uq"].to(wide).view(H, d, self.q_rank)
        uk = tensors["uk"].to(wide).view(H, d, r)
        uv = tensors["uv"].to(wide).view(H, vd, r)
        wo = tensors["o"].to(wide).view(self.hidden, H, vd)
        keep = tensors["uq"].dtype
        rp = self.rank_pad
        w_qk = torch.zeros((H, rp, self.q_rank), dtype=wide, device=uq.device)
        w_qk[:, :r] = torch.einsum("hdr,hdq->hrq", uk, uq)
        w_ov = torch.zeros((self.hidden, H, rp), dtype=wide, device=uq.device)
        w_ov[:, :, :r] = torch.einsum("whv,hvr->whr", wo, uv)
        self.w_qk = w_qk.reshape(H * rp, self.q_rank).to(keep).contiguous()
        self.w_ov = w_ov.reshape(self.hidden, H * rp).to(keep).contiguous()
        self.position.prepare(device)
        why = (ops.attention_refusal(compute_dtype, H, 1, rp) or ops.linear_refusal(self.w_in.dtype, self.hidden))
        if why:
            raise ValueError(f"latent attention mixer: {why}")
        dev = torch.device(device)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
        self._resident = sms * max(1, min(8, 512 // max(1, rp)))

    def weight_bytes(self) -> int:
        ws = (self.w_in, self.w_gate, self.w_qk, self.w_ov, self.norm_q, self.norm_kv)
        return sum(w.numel() * w.element_size() for w in ws)

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(1, self.rank_pad, self.window, values=False)

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, r, rq, rp = self.n_heads, self.kv_rank, self.q_rank, self.rank_pad
        T = x.shape[0]
        new = torch.empty if rp == r else torch.zeros              # columns behind the latent stay zero
        a = project(x, self.w_in)                                           # [T, q_rank + kv_rank]
        cq = torch.empty((T, rq), dtype=a.dtype, device=a.device)
        ops.rmsnorm_cols(a, 0, rq, self.norm_q, self.eps, cq)
        q = project(cq, self.w_qk)                                          # [T, heads * rank]: queries on the latent's side
        if step.mode == "decode":
            # the query rows serve as they are; the latent goes to the cache line and is read from there
            if line.writes:
                kv = new((T, 2 * rp), dtype=a.dtype, device=a.device)             # k | (no v): the append's row layout
                ops.rmsnorm_cols(a, rq, r, self.norm_kv, self.eps, kv)
                ops.cache_append(kv, 0, 1, rp, step.tok_pos, step.tok_slot, line)
            o = self.attend(q, step, line)
        else:
            # packed rows q | c | c: the latent is key and value of the one shared head
            packed = new((T, (H + 2) * rp), dtype=a.dtype, device=a.device)
            ops.copy_cols(q, packed, 0)
            ops.rmsnorm_cols(a, rq, r, self.norm_kv, self.eps, packed, H * rp, (H + 1) * rp)
            if step.mode == "prefill" and line.writes:
                ops.cache_append(packed, H, 1, rp, step.tok_pos, step.tok_slot, line)
            o = self.attend(packed, step, line)
        ops.gate_heads(o, x, self.w_gate, H)                                # times sigmoid(w_g,h . x), float32
        return project(o, self.w_ov)
