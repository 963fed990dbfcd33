"""BERT encoder (post-LayerNorm, learned positions, pooler) written out in
torch.nn: BERT-base has the 199 trainable tensors of the headline gradient set,
BERT-large 391.  Attention uses torch's scaled_dot_product_attention; the model
exists to produce gradients of the right shapes for the data-parallel
benchmarks, with random weights."""
import torch
from torch import nn
from torch.nn import functional as F


class BertLayer(nn.Module):
    def __init__(self, hidden, heads, ffn, dropout):
        super().__init__()
        self.heads = heads
        self.q = nn.Linear(hidden, hidden)
        self.k = nn.Linear(hidden, hidden)
        self.v = nn.Linear(hidden, hidden)
        self.o = nn.Linear(hidden, hidden)
        self.ln1 = nn.LayerNorm(hidden, eps=1e-12)
        self.up = nn.Linear(hidden, ffn)
        self.down = nn.Linear(ffn, hidden)
        self.ln2 = nn.LayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)

    def forward(self, x, mask=None):
        b, s, h = x.shape
        d = h // self.heads

        def split(t):
            return t.view(b, s, self.heads, d).transpose(1, 2)

        a = F.scaled_dot_product_attention(split(self.q(x)), split(self.k(x)), split(self.v(x)),
                                           attn_mask=mask)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x + self.drop(self.o(a)))
        return self.ln2(x + self.drop(self.down(F.gelu(self.up(x)))))


class Bert(nn.Module):
    def __init__(self, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522, max_pos=512,
                 type_vocab=2, dropout=0.1):
        super().__init__()
        self.word = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.segment = nn.Embedding(type_vocab, hidden)
        self.ln = nn.LayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)
        self.layers = nn.ModuleList([BertLayer(hidden, heads, ffn, dropout) for _ in range(layers)])
        self.pooler = nn.Linear(hidden, hidden)

    def forward(self, ids, token_type=None, mask=None):
        """ids: [batch, seq] int64.  Returns (sequence output, pooled output)."""
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device).unsqueeze(0)
        tt = torch.zeros_like(ids) if token_type is None else token_type
        x = self.drop(self.ln(self.word(ids) + self.pos(pos) + self.segment(tt)))
        if mask is not None:  # [batch, seq] of 0/1 -> additive, broadcast over heads and queries
            mask = (1.0 - mask[:, None, None, :].to(x.dtype)) * torch.finfo(x.dtype).min
        for layer in self.layers:
            x = layer(x, mask)
        return x, torch.tanh(self.pooler(x[:, 0]))


def bert_base(**kw):
    return Bert(12, 768, 12, 3072, **kw)


def bert_large(**kw):
    return Bert(24, 1024, 16, 4096, **kw)
