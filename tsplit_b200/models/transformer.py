"""Transformer encoder-decoder (6+6 blocks, d_model 512, 8 heads, FFN 2048,
vocab 32000 by default): shared token embedding, sinusoidal positions, padding
and causal masks, label smoothing — the model of the reference's
``examples/transformer.py:56-287``, with the attention soft-max the reference left
commented out (``transformer.py:156-158``) restored and optional layer norm."""
from __future__ import annotations

import os

import numpy as np

from .. import gpu_ops as ad
from .common import Params


class TransformerConfig(object):
    def __init__(self, vocab_size=32000, d_model=512, num_heads=8, d_ff=2048, num_blocks=6, maxlen1=256,
                 maxlen2=256, dropout_rate=0.0, layer_norm=True, batch_size=8, head_layout=True,
                 fused_softmax=True):
        self.vocab_size, self.d_model, self.num_heads, self.d_ff = vocab_size, d_model, num_heads, d_ff
        self.num_blocks, self.maxlen1, self.maxlen2 = num_blocks, maxlen1, maxlen2
        self.dropout_rate, self.layer_norm, self.batch_size = dropout_rate, layer_norm, batch_size
        #: attention products read / write the [N, T, heads, d] projection layout in place (no head transposes)
        self.head_layout = bool(head_layout) and os.environ.get("TSPLIT_HEAD_LAYOUT", "1") != "0"
        #: scale + padding mask + causal mask + soft-max as one operator (``ad.masked_softmax_op``)
        self.fused_softmax = bool(fused_softmax) and os.environ.get("TSPLIT_FUSED_SOFTMAX", "1") != "0"


class TransformerModel(object):
    def __init__(self, hp, seed=123):
        self.hp = hp
        self.p = Params(seed, scale=0.02)
        self.consts = {}
        self.xs, self.ys_in, self.ys_out = ad.Variable("xs"), ad.Variable("ys_in"), ad.Variable("ys_out")
        self.embeddings = self.p.get("embedding_table", (hp.vocab_size, hp.d_model), scale=hp.d_model ** -0.5)
        self.loss = self._train()
        self.variables = self.p.variables

    # -- helpers ---------------------------------------------------------------
    def const(self, name, value):
        v = ad.Variable(name=name, value=np.asarray(value, dtype=np.float32), trainable=False)
        self.consts[name] = v
        return v

    def dense(self, x, fan_in, fan_out, name, activation=None):
        w = self.p.get(name + "_weight", (fan_in, fan_out), scale=(2.0 / (fan_in + fan_out)) ** 0.5)
        b = self.p.get(name + "_bias", (fan_out,), const=0.0)
        y = ad.matmul_op(x, w)
        y = y + ad.broadcasttoTF_op(b, y)
        return activation(y) if activation is not None else y

    def norm(self, x, name):
        if not self.hp.layer_norm:
            return x
        d = self.hp.d_model
        return ad.layer_normalization_op(x, self.p.get(name + "_ln_scale", (d,), const=1.0),
                                         self.p.get(name + "_ln_bias", (d,), const=0.0))

    def positional(self, tokens, T, maxlen, name):
        hp = self.hp
        E = hp.d_model
        pos = np.array([[q / np.power(10000, (i & -2) / E) for i in range(E)] for q in range(maxlen)])
        pos[:, 0::2] = np.sin(pos[:, 0::2])
        pos[:, 1::2] = np.cos(pos[:, 1::2])
        table = self.const(name + "_position_enc", np.broadcast_to(pos[:T], (hp.batch_size, T, E)))
        return table

    def attention(self, q_in, kv_in, Tq, Tk, name, key_tokens=None, causal=False):
        hp = self.hp
        N, H, d = hp.batch_size, hp.num_heads, hp.d_model
        dh = d // H

        head_layout = getattr(hp, "head_layout", True)

        def heads(x2d, T):
            x = ad.array_reshape_op(x2d, (N, T, H, dh))
            # head layout: the batched products read the projection output [N, T, H, dh] in place; otherwise the
            # heads are transposed to the front as in the reference's example
            return x if head_layout else ad.transpose_op(x, (0, 2, 1, 3))
        q2 = ad.array_reshape_op(q_in, (-1, d))
        k2 = ad.array_reshape_op(kv_in, (-1, d))
        q = heads(self.dense(q2, d, d, name + "_q"), Tq)
        k = heads(self.dense(k2, d, d, name + "_k"), Tk)
        v = heads(self.dense(k2, d, d, name + "_v"), Tk)
        scores = ad.batch_matmul_op(q, k, trans_B=True, heads_A=head_layout, heads_B=head_layout)   # (N, H, Tq, Tk)
        scale = 1.0 / np.sqrt(float(dh))
        if getattr(hp, "fused_softmax", True):
            # scale, key-padding mask (token id 0), causal mask and soft-max in one pass over the scores
            probs = ad.masked_softmax_op(scores, key_tokens, scale=scale, causal=causal)
        else:
            scores = scores * scale
            if key_tokens is not None:            # padding mask: token id 0 is padding
                zeros = ad.zeroslike_op(key_tokens)
                neg = ad.addbyconst_op(zeros, -1e9)
                mask = ad.array_reshape_op(ad.where_op(key_tokens, zeros, neg), (N, 1, 1, Tk))
                scores = scores + ad.broadcasttoTF_op(mask, scores)
            if causal:
                tril = self.const(name + "_tril", np.tril(np.ones((Tq, Tk))))
                future = ad.broadcast_shape_op(tril, (N, H, Tq, Tk))
                neg = ad.addbyconst_op(ad.zeroslike_op(scores), -1e9)
                scores = ad.where_op(future, scores, neg)
            probs = ad.softmax_op(scores)
        if hp.dropout_rate:
            probs = ad.dropout_op(probs, 1.0 - hp.dropout_rate)
        if head_layout:
            ctx = ad.batch_matmul_op(probs, v, heads_B=True, heads_out=True)                # (N, Tq, H, dh)
        else:
            ctx = ad.transpose_op(ad.batch_matmul_op(probs, v), (0, 2, 1, 3))
        out = ad.array_reshape_op(ctx, (N, Tq, d))
        out = ad.array_reshape_op(self.dense(ad.array_reshape_op(out, (-1, d)), d, d, name + "_o"), (N, Tq, d))
        return self.norm(out + q_in, name)

    def ff(self, x, T, name):
        hp = self.hp
        h = ad.array_reshape_op(x, (-1, hp.d_model))
        h = self.dense(h, hp.d_model, hp.d_ff, name + "_ff1", activation=ad.relu_op)
        h = self.dense(h, hp.d_ff, hp.d_model, name + "_ff2")
        return self.norm(ad.array_reshape_op(h, (hp.batch_size, T, hp.d_model)) + x, name + "_ff")

    def embed(self, tokens, T, maxlen, name):
        e = ad.embedding_lookup_op(self.embeddings, tokens) * (self.hp.d_model ** 0.5)
        return e + self.positional(tokens, T, maxlen, name)

    # -- model -----------------------------------------------------------------------
    def _train(self):
        hp = self.hp
        T1, T2 = hp.maxlen1, hp.maxlen2 - 1
        enc = self.embed(self.xs, T1, hp.maxlen1, "enc")
        for i in range(hp.num_blocks):
            enc = self.attention(enc, enc, T1, T1, "enc%d_self" % i, key_tokens=self.xs)
            enc = self.ff(enc, T1, "enc%d" % i)
        dec = self.embed(self.ys_in, T2, hp.maxlen2, "dec")
        for i in range(hp.num_blocks):
            dec = self.attention(dec, dec, T2, T2, "dec%d_self" % i, key_tokens=self.ys_in, causal=True)
            dec = self.attention(dec, enc, T2, T1, "dec%d_cross" % i, key_tokens=self.xs)
            dec = self.ff(dec, T2, "dec%d" % i)
        logits = ad.matmul_op(ad.array_reshape_op(dec, (-1, hp.d_model)), self.embeddings, trans_B=True)
        self.logits = logits
        onehot = ad.array_reshape_op(ad.one_hot_op(self.ys_out, hp.vocab_size), (-1, hp.vocab_size))
        eps = 0.1
        smooth = ad.addbyconst_op(ad.mul_byconst_op(onehot, 1 - eps), eps / hp.vocab_size)
        return ad.softmaxcrossentropy_op(logits, smooth)

    def synthetic_batch(self, seed=0):
        hp = self.hp
        r = np.random.RandomState(seed)
        xs = r.randint(1, hp.vocab_size, (hp.batch_size, hp.maxlen1)).astype(np.float32)
        ys = r.randint(1, hp.vocab_size, (hp.batch_size, hp.maxlen2)).astype(np.float32)
        return {self.xs: xs, self.ys_in: ys[:, :-1].copy(), self.ys_out: ys[:, 1:].copy()}

    def tokens_per_step(self):
        return self.hp.batch_size * (self.hp.maxlen1 + self.hp.maxlen2 - 1)


def transformer(**kw):
    seed = kw.pop("seed", 123)
    return TransformerModel(TransformerConfig(**kw), seed=seed)
