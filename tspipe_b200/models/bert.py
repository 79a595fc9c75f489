"""BERT / DistilBERT encoders as cut-able ``nn.Sequential``s for masked-LM distillation.

The reference converts Hugging Face ``BertForMaskedLM`` / ``DistilBertForMaskedLM`` into sequentials of
``TSPipeModelWrapper`` ed blocks that pass 16- / 9-element lists between stages
(`benchmarks/distilbert/bert.py:12-61,104-266`, `benchmarks/distilbert/distillbert.py:18-195`).  These are
self-contained re-implementations with the same architecture and the same stage interface idea: every
stage takes and returns a pytree ``{"hidden": [B, L, H], "mask": [B, L]}`` (the padding mask rides along
untouched, without a gradient), wrapped in :class:`~tspipe_b200.model_wrapper.TSPipeModelWrapper`, and the
last child returns ``(mlm_logits [B, L, V], last_hidden [B, L, H])`` - what the distillation loss needs
(`benchmarks/distilbert/distiller.py:711-772`).

Differences from the HF modules, by design: the MLM decoder is not weight-tied to the word embeddings (they
live on different pipeline stages), attention is the fused op of :mod:`tspipe_b200.ops.attention`,
LayerNorm / bias+GELU are the fused kernels.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..model_wrapper import TSPipeModelWrapper
from ..ops import fused
from ..ops.attention import attention, project_qkv
from ..ops.linear import linear
from .vit import LayerNorm


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    max_pos: int = 512
    type_vocab: int = 2
    eps: float = 1e-12
    dropout: float = 0.1
    distil: bool = False        # DistilBERT: no token-type embeddings


BERT_BASE = BertConfig()
DISTILBERT_BASE = BertConfig(layers=6, distil=True)
BERT_LARGE = BertConfig(hidden=1024, layers=24, heads=16, ffn=4096)
BERT_TINY_TEST = BertConfig(vocab_size=128, hidden=32, layers=2, heads=4, ffn=64, max_pos=32, dropout=0.0)
DISTIL_TINY_TEST = BertConfig(vocab_size=128, hidden=32, layers=1, heads=4, ffn=64, max_pos=32, dropout=0.0, distil=True)


class Embeddings(nn.Module):
    """Input: ``{"input_ids": [B, L] int64, "attention_mask": [B, L]}``; output ``{"hidden", "mask"}``."""

    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.word = nn.Embedding(cfg.vocab_size, cfg.hidden)
        self.pos = nn.Embedding(cfg.max_pos, cfg.hidden)
        self.tok_type = None if cfg.distil else nn.Embedding(cfg.type_vocab, cfg.hidden)
        self.norm = LayerNorm(cfg.hidden, eps=cfg.eps)
        self.drop = nn.Dropout(cfg.dropout)

    def forward(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        ids = batch["input_ids"]
        mask = batch["attention_mask"]
        pos = torch.arange(ids.shape[1], device=ids.device)
        h = self.word(ids) + self.pos(pos)[None]
        if self.tok_type is not None:
            h = h + self.tok_type.weight[0]
        return {"hidden": self.drop(self.norm(h)), "mask": mask}


class EncoderLayer(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.heads = cfg.heads
        self.qkv = nn.Linear(cfg.hidden, 3 * cfg.hidden)
        self.out = nn.Linear(cfg.hidden, cfg.hidden)
        self.norm1 = LayerNorm(cfg.hidden, eps=cfg.eps)
        self.fc1 = nn.Linear(cfg.hidden, cfg.ffn)
        self.fc2 = nn.Linear(cfg.ffn, cfg.hidden)
        self.norm2 = LayerNorm(cfg.hidden, eps=cfg.eps)
        self.drop = nn.Dropout(cfg.dropout)

    def forward(self, s: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        x, mask = s["hidden"], s["mask"]
        b, l, c = x.shape
        q, k, v = project_qkv(x, self.qkv.weight, self.qkv.bias, self.heads)
        key_mask = mask.to(torch.bool)[:, None, None, :]
        a = attention(q, k, v, key_mask).transpose(1, 2).reshape(b, l, c)
        x = self.norm1(x + self.drop(linear(a, self.out.weight, self.out.bias)))
        h = fused.gelu(linear(x, self.fc1.weight, None), self.fc1.bias)
        x = self.norm2(x + self.drop(linear(h, self.fc2.weight, self.fc2.bias)))
        return {"hidden": x, "mask": mask}


class MlmHead(nn.Module):
    """Transform (dense + GELU + LayerNorm) and vocabulary projection; returns ``(logits, last_hidden)``.  On CUDA
    the class dimension of the logits is padded to a multiple of 8 with classes of probability zero."""

    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.dense = nn.Linear(cfg.hidden, cfg.hidden)
        self.norm = LayerNorm(cfg.hidden, eps=cfg.eps)
        self.decoder = nn.Linear(cfg.hidden, cfg.vocab_size)

    def forward(self, s: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        x = s["hidden"]
        h = self.norm(fused.gelu(linear(x, self.dense.weight, None), self.dense.bias))
        w, b = self.decoder.weight, self.decoder.bias
        pad = (-w.shape[0]) % 8
        if h.is_cuda and pad:
            # A vocabulary of 30 522 entries is no multiple of 8 elements, which sends this GEMM and its two
            # backward products to the library's unaligned fallback kernels (2.8 ms instead of 0.8 ms for 16 K
            # tokens).  Pad the classes: the extra ones get a bias of -30000, so their probability is exactly zero in
            # every softmax (student and teacher alike) and they receive no gradient.
            w = F.pad(w, (0, 0, 0, pad))
            b = F.pad(b, (0, pad), value=-30000.0)
        return linear(h, w, b), x


def bert_mlm_sequential(cfg: BertConfig) -> nn.Sequential:
    """Children: embeddings, one per encoder layer, MLM head - each wrapped for pytree stage I/O."""
    ch: "OrderedDict[str, nn.Module]" = OrderedDict()
    ch["embeddings"] = TSPipeModelWrapper(Embeddings(cfg))
    for i in range(cfg.layers):
        ch[f"layer{i}"] = TSPipeModelWrapper(EncoderLayer(cfg))
    ch["mlm_head"] = TSPipeModelWrapper(MlmHead(cfg))
    seq = nn.Sequential(ch)
    for m in seq.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)
    return seq


def distillation_pair(teacher_cfg: BertConfig = BERT_BASE, student_cfg: BertConfig = DISTILBERT_BASE
                      ) -> Tuple[nn.Sequential, nn.Sequential]:
    """``(student, teacher)``; the student's layers are initialised from every other teacher layer, as the
    reference's extraction script does for DistilBERT."""
    teacher = bert_mlm_sequential(teacher_cfg)
    student = bert_mlm_sequential(student_cfg)
    if teacher_cfg.hidden == student_cfg.hidden and teacher_cfg.ffn == student_cfg.ffn:
        step = max(teacher_cfg.layers // max(student_cfg.layers, 1), 1)
        with torch.no_grad():
            for i in range(student_cfg.layers):
                src = getattr(teacher, f"layer{min(i * step, teacher_cfg.layers - 1)}").state_dict()
                getattr(student, f"layer{i}").load_state_dict(src)
    return student, teacher
