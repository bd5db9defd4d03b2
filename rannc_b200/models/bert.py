"""BERT for masked-LM + next-sentence pre-training (post-LN encoder, GELU FFN).

Plain ``torch.nn`` code with no dependency on the rest of the package: the
middleware traces it like any other user model.  The configurations used by the
benchmarks are BERT-Large (24 x 1024, 16 heads) and its enlarged variants
(256 x 2048 and 128 x 4096).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12
    # rows of the (tied) word-embedding / decoder matrix are padded to a multiple of this, so that
    # the decoder GEMM operands have 16-byte aligned rows; padded logits never enter the loss
    pad_vocab_to: int = 64

    @property
    def padded_vocab_size(self) -> int:
        m = max(1, self.pad_vocab_to)
        return (self.vocab_size + m - 1) // m * m

    @staticmethod
    def large(**kw) -> "BertConfig":
        return BertConfig(**kw)

    @staticmethod
    def base(**kw) -> "BertConfig":
        return BertConfig(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072, **kw)

    @staticmethod
    def enlarged_13b(**kw) -> "BertConfig":
        return BertConfig(hidden_size=2048, num_hidden_layers=256, num_attention_heads=32, intermediate_size=8192, **kw)

    @staticmethod
    def enlarged_26b(**kw) -> "BertConfig":
        return BertConfig(hidden_size=4096, num_hidden_layers=128, num_attention_heads=64, intermediate_size=16384,
                          **kw)

    @staticmethod
    def tiny(**kw) -> "BertConfig":
        d = dict(vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                 intermediate_size=1024, max_position_embeddings=128)
        d.update(kw)
        return BertConfig(**d)


class BertEmbeddings(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(cfg.padded_vocab_size, cfg.hidden_size)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.token_type_embeddings = nn.Embedding(cfg.type_vocab_size, cfg.hidden_size)
        self.LayerNorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)
        self.register_buffer("position_ids", torch.arange(cfg.max_position_embeddings).unsqueeze(0),
                             persistent=False)

    def forward(self, input_ids, token_type_ids):
        S = input_ids.shape[1]
        pos = self.position_ids[:, :S]
        x = self.word_embeddings(input_ids) + self.position_embeddings(pos) + self.token_type_embeddings(token_type_ids)
        return self.dropout(self.LayerNorm(x))


class BertSelfAttention(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.h = cfg.num_attention_heads
        self.d = cfg.hidden_size // cfg.num_attention_heads
        self.query = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.key = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.value = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.p = cfg.attention_probs_dropout_prob

    def forward(self, x, attn_bias):
        B, S, _ = x.shape
        q = self.query(x).view(B, S, self.h, self.d).transpose(1, 2)
        k = self.key(x).view(B, S, self.h, self.d).transpose(1, 2)
        v = self.value(x).view(B, S, self.h, self.d).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_bias, dropout_p=self.p if self.training else 0.0)
        return o.transpose(1, 2).reshape(B, S, self.h * self.d)


class BertLayer(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.attention = BertSelfAttention(cfg)
        self.attn_out = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.attn_dropout = nn.Dropout(cfg.hidden_dropout_prob)
        self.attn_ln = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.ffn_in = nn.Linear(cfg.hidden_size, cfg.intermediate_size)
        self.ffn_out = nn.Linear(cfg.intermediate_size, cfg.hidden_size)
        self.ffn_dropout = nn.Dropout(cfg.hidden_dropout_prob)
        self.ffn_ln = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)

    def forward(self, x, attn_bias):
        a = self.attention(x, attn_bias)
        x = self.attn_ln(self.attn_dropout(self.attn_out(a)) + x)
        f = self.ffn_out(F.gelu(self.ffn_in(x)))
        return self.ffn_ln(self.ffn_dropout(f) + x)


class BertModel(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.cfg = cfg
        self.embeddings = BertEmbeddings(cfg)
        self.layers = nn.ModuleList([BertLayer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.pooler = nn.Linear(cfg.hidden_size, cfg.hidden_size)

    def forward(self, input_ids, token_type_ids, attention_mask):
        # additive key bias, broadcast over heads and queries
        bias = (1.0 - attention_mask[:, None, None, :].to(self.pooler.weight.dtype)) * -10000.0
        x = self.embeddings(input_ids, token_type_ids)
        for layer in self.layers:
            x = layer(x, bias)
        pooled = torch.tanh(self.pooler(x[:, 0]))
        return x, pooled


class BertForPreTraining(nn.Module):
    """Returns the scalar pre-training loss: masked-LM cross entropy + next-sentence cross entropy."""

    def __init__(self, cfg: BertConfig, init_weights: bool = True):
        """``init_weights=False`` keeps the layers' own default initialisation (needed when the parameters no
        longer hold their full values at this point, e.g. when they are sharded as they are constructed)."""
        super().__init__()
        self.cfg = cfg
        self.bert = BertModel(cfg)
        self.transform = nn.Linear(cfg.hidden_size, cfg.hidden_size)
        self.transform_ln = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.decoder_bias = nn.Parameter(torch.zeros(cfg.padded_vocab_size))
        self.seq_relationship = nn.Linear(cfg.hidden_size, 2)
        if init_weights:
            self.apply(self._init)

    def _init(self, m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)

    def forward(self, input_ids, token_type_ids, attention_mask, masked_lm_labels, next_sentence_label):
        x, pooled = self.bert(input_ids, token_type_ids, attention_mask)
        h = self.transform_ln(F.gelu(self.transform(x)))
        # decoder weight tied to the word embeddings
        logits = F.linear(h, self.bert.embeddings.word_embeddings.weight, self.decoder_bias)
        V = self.cfg.vocab_size
        mlm = F.cross_entropy(logits[..., :V].reshape(-1, V).float(), masked_lm_labels.reshape(-1), ignore_index=-100)
        nsp = F.cross_entropy(self.seq_relationship(pooled).float(), next_sentence_label.reshape(-1))
        return mlm + nsp


def synthetic_batch(cfg: BertConfig, batch: int, seq: int, device="cpu", seed: int = 0, mask_prob: float = 0.15):
    """Token ids uniform over the vocabulary, 15 % of positions as MLM labels, NSP labels Bernoulli(0.5)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=g)
    tt = torch.zeros(batch, seq, dtype=torch.long)
    tt[:, seq // 2:] = 1
    mask = torch.ones(batch, seq, dtype=torch.long)
    labels = torch.full((batch, seq), -100, dtype=torch.long)
    sel = torch.rand(batch, seq, generator=g) < mask_prob
    labels[sel] = ids[sel]
    nsp = (torch.rand(batch, generator=g) < 0.5).long()
    return tuple(t.to(device) for t in (ids, tt, mask, labels, nsp))
