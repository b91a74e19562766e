"""GPT-2 as pipeline stages of tensor-parallel, sequence-parallel transformer blocks.

One ``GPT2Stage`` is what one rank holds: a contiguous range of blocks, sharded ``tp.n`` ways, plus
the embeddings on the first stage and the final norm, LM head and loss on the last.  Activations
between blocks are sharded along the token dimension (every rank keeps ``tokens / tp.n`` rows), so the
layer norms, residuals and dropouts never repeat work; a block's two GEMM pairs are

    all-gather -> GEMM (q/k/v)   ... attention on the local heads ...   GEMM -> reduce-scatter (out)
    all-gather -> GEMM (4d up)   ... GELU ...                           GEMM -> reduce-scatter (down)

each pair member one fused tcgen05 kernel (``dfccl_b200.parallel.tp``).  Attention itself is the
library kernel behind ``scaled_dot_product_attention``.

The reference ships no model code; its simulator only knows the communication group structure of
such a job (reference: simulator/simulator.py:434-493, simulator/configs/megatron.json).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.fused_linear import TpGroup
from ..parallel.tp import ColumnParallelLinear, RowParallelLinear


@dataclass
class GPT2Config:
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    seq_len: int = 1024
    vocab: int = 50257
    init_std: float = 0.02

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=4, d_model=256, n_head=4, seq_len=128, vocab=512)

    def n_params(self) -> int:
        d = self.d_model
        return self.n_layer * (12 * d * d + 13 * d) + (self.vocab + self.seq_len) * d + 2 * d


def _full(shape, std: float, seed: int, device) -> torch.Tensor:
    """The unsharded weight: the same values on every rank (seeded on the CPU generator), then sliced."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(device)


def _replicated(m: nn.Module) -> nn.Module:
    for p in m.parameters():
        p.tp_replicated = True
    return m


class ParallelBlock(nn.Module):
    def __init__(self, cfg: GPT2Config, tp: TpGroup, tokens: int, layer: int, seed: int):
        super().__init__()
        d, dev = cfg.d_model, tp.device
        assert cfg.n_head % tp.n == 0 and tokens % tp.n == 0
        self.cfg, self.tp, self.tokens = cfg, tp, tokens
        self.heads_local = cfg.n_head // tp.n
        rows = tokens // tp.n
        s = seed + 16 * layer
        self.ln1 = _replicated(nn.LayerNorm(d, dtype=torch.bfloat16, device=dev))
        self.qkv = ColumnParallelLinear(tp, rows, _full((3 * d, d), cfg.init_std, s + 1, dev), parts=3)
        self.proj = RowParallelLinear(tp, tokens, _full((d, d), cfg.init_std / (2 * cfg.n_layer) ** 0.5, s + 2, dev))
        self.ln2 = _replicated(nn.LayerNorm(d, dtype=torch.bfloat16, device=dev))
        self.up = ColumnParallelLinear(tp, rows, _full((4 * d, d), cfg.init_std, s + 3, dev))
        self.down = RowParallelLinear(tp, tokens, _full((d, 4 * d), cfg.init_std / (2 * cfg.n_layer) ** 0.5, s + 4, dev))

    def forward(self, h: torch.Tensor) -> torch.Tensor:          # [tokens / tp, d]
        cfg = self.cfg
        hd = cfg.d_model // cfg.n_head
        b = self.tokens // cfg.seq_len
        qkv = self.qkv(self.ln1(h)).view(b, cfg.seq_len, 3, self.heads_local, hd)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))     # [b, heads, seq, hd]
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        h = h + self.proj(a.transpose(1, 2).reshape(self.tokens, self.heads_local * hd))
        return h + self.down(F.gelu(self.up(self.ln2(h)), approximate="tanh"))


class GPT2Stage(nn.Module):
    """Blocks ``[first_layer, first_layer + n_layers)`` of the model for micro-batches of
    ``micro_batch`` sequences."""

    def __init__(self, cfg: GPT2Config, tp: TpGroup, stage: int, n_stages: int, micro_batch: int, seed: int = 1234):
        super().__init__()
        assert cfg.n_layer % n_stages == 0
        self.cfg, self.tp = cfg, tp
        self.is_first, self.is_last = stage == 0, stage == n_stages - 1
        self.tokens = micro_batch * cfg.seq_len
        self.rows = self.tokens // tp.n
        per = cfg.n_layer // n_stages
        dev, d = tp.device, cfg.d_model
        if self.is_first:
            self.wte = _replicated(nn.Embedding(cfg.vocab, d, dtype=torch.bfloat16, device=dev))
            self.wpe = _replicated(nn.Embedding(cfg.seq_len, d, dtype=torch.bfloat16, device=dev))
            with torch.no_grad():
                self.wte.weight.copy_(_full((cfg.vocab, d), cfg.init_std, seed + 7, dev))
                self.wpe.weight.copy_(_full((cfg.seq_len, d), cfg.init_std, seed + 8, dev))
            pos = torch.arange(self.tokens, device=dev) % cfg.seq_len
            self.register_buffer("pos", pos[tp.rank * self.rows:(tp.rank + 1) * self.rows], persistent=False)
        self.blocks = nn.ModuleList(ParallelBlock(cfg, tp, self.tokens, stage * per + i, seed + 1000)
                                    for i in range(per))
        if self.is_last:
            self.ln_f = _replicated(nn.LayerNorm(d, dtype=torch.bfloat16, device=dev))
            # the output projection is a parameter of its own (not tied to the embedding of another stage)
            self.head = nn.Parameter(_full((cfg.vocab, d), cfg.init_std, seed + 9, dev).to(torch.bfloat16))
            self.head.tp_replicated = True

    def my_rows(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.tp.rank * self.rows:(self.tp.rank + 1) * self.rows]

    def forward(self, x: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        """First stage: ``x`` are token ids [micro_batch, seq]; later stages: hidden rows [tokens / tp, d].
        The last stage returns this rank's share of the mean token loss (the shares of a group add up
        to the micro-batch's loss); the others return their hidden rows."""
        if self.is_first:
            ids = self.my_rows(x.reshape(-1))
            h = self.wte(ids) + self.wpe(self.pos)
        else:
            h = x
        for blk in self.blocks:
            h = blk(h)
        if not self.is_last:
            return h
        logits = self.ln_f(h) @ self.head.t()
        return F.cross_entropy(logits.float(), self.my_rows(targets.reshape(-1)), reduction="sum") / self.tokens
