"""A PCF-NAT-style embedding extractor built on the fused neighbourhood-attention layer.

This is the model-level workload of the benchmark suite (80-dim log-mel input -> Conv1d 80->256 -> 6 stages x 4
neighbourhood-attention transformer blocks with progressive channel fusion -> attentive statistics pooling -> 192-d
embedding -> AAM-softmax), written from its description, channels-last so that every projection is one GEMM on
``(N*T, C)`` and the attention layer needs no transposing copies around its projections. It follows the structure of
the reference's ``models/PCF_NATransformer.py`` (stages of NA blocks whose outputs are concatenated along channels and
fused by a 1x1 projection; ``:228-303`` layers and blocks, ``:319-455`` the network) but is not state-dict compatible
with it: weights are random-init, which is all a throughput benchmark needs. The attention layers are
``pcf_nat_b200.NAttention`` (``layout="channels_last"``).

``attention="unfused"`` swaps in the reference's own operator sequence -- ``q*scale -> QK -> +rpb -> softmax -> AV`` through
the drop-in ``getNA1dFunction`` pair with the fp32 ``(N*heads, T, win)`` tensor in HBM -- for an A/B of the fused layer
inside a whole training step.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .nattention import NAttention, _merge_heads, _split_heads
from .nattn import getNA1dFunction


class UnfusedNAttention(NAttention):
    """Same parameters as ``NAttention``; forward runs the reference's unfused chain (PCF_NATransformer.py:141-150)."""

    def forward(self, x, padding=None):
        layout = self._na1d_layout
        N = x.shape[0]
        T = x.shape[2] if layout == "channels_first" else x.shape[1]
        q, k, v = _split_heads(self.qkv(x), layout, self.num_heads, self.groups)
        QK, AV = getNA1dFunction(q.shape[-1], self.dilation, q.dtype)
        attn = QK.apply(q * self.scale, k, self.win_size, self.left, self.dilation)
        attn = attn.view(N, self.num_heads, T, self.win_size) + self.relative_position_bias
        attn = attn + self.attn_mask.to(attn.dtype)
        attn = attn.view(N * self.num_heads, T, self.win_size).softmax(dim=-1)
        o = AV.apply(attn, v, self.win_size, self.left, self.dilation)
        return self.proj_drop(self.proj(_merge_heads(o, layout, N, self.num_heads)))


def _layer_norm(x, ln):
    """LayerNorm on the activation's own dtype. Under autocast PyTorch runs layer_norm in fp32 (a cast of the 16-bit
    residual stream up, an fp32 kernel, and a cast back down for the next projection); the 16-bit kernel (16-bit in/out and
    parameters, fp32 statistics) does the same arithmetic with a third of the traffic."""
    if x.dtype in (torch.bfloat16, torch.float16) and torch.is_autocast_enabled():
        with torch.autocast(x.device.type, enabled=False):
            return F.layer_norm(x, ln.normalized_shape, ln.weight.to(x.dtype), ln.bias.to(x.dtype), ln.eps)
    return ln(x)


class NABlock(nn.Module):
    """x + NA(LN(x)); x + MLP(LN(x)) on (N, T, C)."""

    def __init__(self, frames, dim, heads, win, mlp_ratio, attention):
        super().__init__()
        cls = NAttention if attention == "fused" else UnfusedNAttention
        self.norm1 = nn.LayerNorm(dim)
        self.attn = cls(frames, dim, heads, win, layout="channels_last")
        self.norm2 = nn.LayerNorm(dim)
        self.fc1 = nn.Linear(dim, dim * mlp_ratio)
        self.fc2 = nn.Linear(dim * mlp_ratio, dim)

    def forward(self, x, padding=None):
        x = x + self.attn(_layer_norm(x, self.norm1), padding)
        return x + self.fc2(F.gelu(self.fc1(_layer_norm(x, self.norm2))))


class AttentiveStatsPool(nn.Module):
    """Channel-wise attention over time -> weighted mean and standard deviation, (N, T, C) -> (N, 2C)."""

    def __init__(self, dim, bottleneck=128):
        super().__init__()
        self.a = nn.Linear(dim, bottleneck)
        self.b = nn.Linear(bottleneck, dim)

    def forward(self, x):
        w = torch.softmax(self.b(torch.tanh(self.a(x))).float(), dim=1)
        xf = x.float()
        mu = (w * xf).sum(1)
        var = (w * xf * xf).sum(1) - mu * mu
        return torch.cat([mu, var.clamp_min(1e-5).sqrt()], dim=1)


class AAMSoftmax(nn.Module):
    """Additive angular margin softmax loss over `classes` (cos(theta + m) on the target logit, scale s)."""

    def __init__(self, dim, classes, margin=0.2, scale=30.0):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(classes, dim) * 0.01)
        self.m, self.s = margin, scale

    def forward(self, emb, labels):
        with torch.autocast(emb.device.type, enabled=False):  # the margin arithmetic stays in fp32
            return self._loss(emb.float(), labels)

    def _loss(self, emb, labels):
        cos = F.linear(F.normalize(emb.float()), F.normalize(self.weight.float())).clamp(-1 + 1e-7, 1 - 1e-7)
        target = torch.cos(torch.acos(cos.gather(1, labels[:, None])) + self.m)
        logits = cos.scatter(1, labels[:, None], target) * self.s
        return F.cross_entropy(logits, labels)


class PCFNATExtractor(nn.Module):
    def __init__(self, frames=300, feat=80, dim=256, heads=4, win=7, stages=6, blocks=4, mlp_ratio=4, emb=192,
                 classes=5994, attention="fused"):
        super().__init__()
        if attention not in ("fused", "unfused"):
            raise ValueError("attention must be 'fused' or 'unfused'")
        self.front = nn.Conv1d(feat, dim, kernel_size=5, padding=2)
        self.stages = nn.ModuleList(nn.ModuleList(NABlock(frames, dim, heads, win, mlp_ratio, attention) for _ in range(blocks))
                                    for _ in range(stages))
        # progressive channel fusion: the input of stage s+1 is a 1x1 projection of the concatenated outputs of stages <= s
        self.fuse = nn.ModuleList(nn.Linear((s + 2) * dim, dim) for s in range(stages - 1))
        self.pool = AttentiveStatsPool(stages * dim)
        self.bn = nn.BatchNorm1d(2 * stages * dim)
        self.embed = nn.Linear(2 * stages * dim, emb)
        self.loss = AAMSoftmax(emb, classes)

    def embedding(self, fbank, padding=None):
        x = self.front(fbank).transpose(1, 2).contiguous()  # (N, T, C)
        feats = [x]
        outs = []
        for s, stage in enumerate(self.stages):
            for blk in stage:
                x = blk(x, padding)
            outs.append(x)
            feats.append(x)
            if s + 1 < len(self.stages):
                x = self.fuse[s](torch.cat(feats, dim=-1))
        pooled = self.pool(torch.cat(outs, dim=-1))
        return self.embed(self.bn(pooled).to(self.embed.weight.dtype))

    def forward(self, fbank, labels, padding=None):
        return self.loss(self.embedding(fbank, padding), labels)


def model_flops_per_utterance(frames=300, feat=80, dim=256, stages=6, blocks=4, mlp_ratio=4, emb=192, classes=5994, win=7):
    """Forward+backward (3x forward) matmul FLOPs per utterance, for the fraction-of-tensor-peak figure."""
    per_tok_block = 2 * dim * 3 * dim + 2 * dim * dim + 2 * 2 * dim * dim * mlp_ratio + 4 * win * dim
    body = stages * blocks * per_tok_block * frames
    fuse = sum(2 * (s + 2) * dim * dim for s in range(stages - 1)) * frames
    front = 2 * feat * dim * 5 * frames
    pool = (2 * stages * dim * 128 * 2) * frames
    head = 2 * 2 * stages * dim * emb + 2 * emb * classes
    return 3 * (body + fuse + front + pool + head)
