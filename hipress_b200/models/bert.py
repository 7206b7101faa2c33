"""BERT-large (24 layers, hidden 1024, 16 heads, FFN 4096, vocab 30522) with a
masked-language-model head, for the onebit / CaSync-Ring configuration."""

import torch
import torch.nn as nn
import torch.nn.functional as F


class BertConfig:
    def __init__(self, vocab_size=30522, hidden=1024, layers=24, heads=16, ffn=4096,
                 max_pos=512, type_vocab=2, dropout=0.1):
        self.vocab_size, self.hidden, self.layers, self.heads = vocab_size, hidden, layers, heads
        self.ffn, self.max_pos, self.type_vocab, self.dropout = ffn, max_pos, type_vocab, dropout


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.heads = c.heads
        self.qkv = nn.Linear(c.hidden, 3 * c.hidden)
        self.proj = nn.Linear(c.hidden, c.hidden)
        self.ln1 = nn.LayerNorm(c.hidden, eps=1e-12)
        self.fc1 = nn.Linear(c.hidden, c.ffn)
        self.fc2 = nn.Linear(c.ffn, c.hidden)
        self.ln2 = nn.LayerNorm(c.hidden, eps=1e-12)
        self.drop = nn.Dropout(c.dropout)
        self.p = c.dropout

    def forward(self, x):
        B, S, H = x.shape
        q, k, v = self.qkv(x).view(B, S, 3, self.heads, H // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, dropout_p=self.p if self.training else 0.0)
        a = a.transpose(1, 2).reshape(B, S, H)
        x = self.ln1(x + self.drop(self.proj(a)))
        return self.ln2(x + self.drop(self.fc2(F.gelu(self.fc1(x)))))


class BertForMaskedLM(nn.Module):
    def __init__(self, c: BertConfig | None = None):
        super().__init__()
        c = c or BertConfig()
        self.c = c
        self.tok = nn.Embedding(c.vocab_size, c.hidden)
        self.pos = nn.Embedding(c.max_pos, c.hidden)
        self.typ = nn.Embedding(c.type_vocab, c.hidden)
        self.ln = nn.LayerNorm(c.hidden, eps=1e-12)
        self.drop = nn.Dropout(c.dropout)
        self.layers = nn.ModuleList(BertLayer(c) for _ in range(c.layers))
        self.head_dense = nn.Linear(c.hidden, c.hidden)
        self.head_ln = nn.LayerNorm(c.hidden, eps=1e-12)
        self.head_bias = nn.Parameter(torch.zeros(c.vocab_size))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, ids, labels=None):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)
        x = self.drop(self.ln(self.tok(ids) + self.pos(pos)[None] + self.typ.weight[0][None, None]))
        for l in self.layers:
            x = l(x)
        h = self.head_ln(F.gelu(self.head_dense(x)))
        if labels is None:
            return F.linear(h, self.tok.weight, self.head_bias)
        # score only the masked positions (labels == -100 elsewhere)
        sel = labels.view(-1) != -100
        hs = h.view(-1, h.shape[-1])[sel]
        logits = F.linear(hs, self.tok.weight, self.head_bias)
        return F.cross_entropy(logits.float(), labels.view(-1)[sel])


def bert_large(**kw):
    return BertForMaskedLM(BertConfig(**kw))


def bert_tiny():
    return BertForMaskedLM(BertConfig(vocab_size=1000, hidden=64, layers=2, heads=4, ffn=128, max_pos=64))
