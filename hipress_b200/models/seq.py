"""Sequence models of the HiPress evaluation set beyond BERT-large: BERT-base, a
two-layer LSTM language model and the base encoder-decoder Transformer (the
reference's paper trains them with its MXNet / PyTorch front ends; the mounted tree
names only ``--model vgg19``, README.md:45 of mark14wu/hipress)."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .bert import BertConfig, BertForMaskedLM


def bert_base(**kw):
    cfg = dict(hidden=768, layers=12, heads=12, ffn=3072)
    cfg.update(kw)
    return BertForMaskedLM(BertConfig(**cfg))


class LSTMLanguageModel(nn.Module):
    """Embedding -> 2-layer LSTM -> vocabulary projection (word-level LM)."""

    def __init__(self, vocab_size: int = 33278, emb: int = 1500, hidden: int = 1500, layers: int = 2,
                 dropout: float = 0.5):
        super().__init__()
        self.vocab_size = vocab_size
        self.drop = nn.Dropout(dropout)
        self.embed = nn.Embedding(vocab_size, emb)
        self.lstm = nn.LSTM(emb, hidden, layers, dropout=dropout if layers > 1 else 0.0, batch_first=True)
        self.out = nn.Linear(hidden, vocab_size)
        nn.init.uniform_(self.embed.weight, -0.1, 0.1)
        nn.init.uniform_(self.out.weight, -0.1, 0.1)
        nn.init.zeros_(self.out.bias)

    def forward(self, ids, labels=None):
        h, _ = self.lstm(self.drop(self.embed(ids)))
        logits = self.out(self.drop(h))
        if labels is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, self.vocab_size), labels.view(-1))


class TransformerSeq2Seq(nn.Module):
    """Base Transformer (6 + 6 layers, d_model 512, 8 heads, FFN 2048), shared
    source / target vocabulary and tied output projection."""

    def __init__(self, vocab_size: int = 32000, d_model: int = 512, heads: int = 8, layers: int = 6,
                 ffn: int = 2048, dropout: float = 0.1, max_len: int = 512):
        super().__init__()
        self.vocab_size, self.d_model = vocab_size, d_model
        self.embed = nn.Embedding(vocab_size, d_model)
        pos = torch.arange(max_len)[:, None]
        div = torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2], pe[:, 1::2] = torch.sin(pos * div), torch.cos(pos * div)
        self.register_buffer("pe", pe, persistent=False)
        self.core = nn.Transformer(d_model, heads, layers, layers, ffn, dropout, batch_first=True,
                                   norm_first=True)
        self.drop = nn.Dropout(dropout)
        nn.init.normal_(self.embed.weight, 0.0, d_model ** -0.5)

    def _emb(self, ids):
        return self.drop(self.embed(ids) * math.sqrt(self.d_model) + self.pe[: ids.shape[1]][None])

    def forward(self, src, labels=None):
        """Synthetic-task form: the target is `labels` (teacher forcing with a shifted copy)."""
        tgt_in = src if labels is None else torch.cat([labels[:, :1], labels[:, :-1]], dim=1)
        mask = nn.Transformer.generate_square_subsequent_mask(tgt_in.shape[1], device=src.device)
        h = self.core(self._emb(src), self._emb(tgt_in), tgt_mask=mask, tgt_is_causal=True)
        logits = F.linear(h, self.embed.weight)
        if labels is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, self.vocab_size), labels.view(-1))


def lstm_lm(**kw):
    return LSTMLanguageModel(**kw)


def transformer_base(**kw):
    return TransformerSeq2Seq(**kw)
