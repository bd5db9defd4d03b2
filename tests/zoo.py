"""Small models that each exercise one graph shape the partitioner must cope with: conv + fc, fork/join,
shared (fan-out) activations, tied weights, scalar-loss output, integer inputs, mixed LayerNorm, BatchNorm
buffers, tiny parameters, tensor constants, parameter-free graphs, an unrolled helper loop, read-only and
overwritten buffers.  Same coverage as the reference's test zoo (test/models.py), written independently."""
import torch
import torch.nn as nn
import torch.nn.functional as F


class Basic(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(1, 4, 3, padding=1)
        self.c2 = nn.Conv2d(4, 8, 3, padding=1)
        self.f1 = nn.Linear(8 * 4 * 4, 32)
        self.f2 = nn.Linear(32, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return self.f2(F.relu(self.f1(x.flatten(1))))


class ForkJoin(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(16, 16)
        self.b1 = nn.Linear(16, 16)
        self.b2 = nn.Linear(16, 16)
        self.c = nn.Linear(16, 8)

    def forward(self, x):
        h = torch.relu(self.a(x))
        return self.c(torch.relu(self.b1(h)) + torch.tanh(self.b2(h)))


class SharedInput(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 16)
        self.l2 = nn.Linear(16, 16)
        self.l3 = nn.Linear(16, 16)

    def forward(self, x):
        h = self.l1(x)
        return self.l3(torch.relu(self.l2(h)) + h) + x


class SharedParam(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 16)
        self.mid = nn.Linear(16, 16)

    def forward(self, x):
        return self.l1(torch.relu(self.mid(torch.relu(self.l1(x)))))


class LossOut(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 32)
        self.l2 = nn.Linear(32, 32)
        self.l3 = nn.Linear(32, 5)

    def forward(self, x, y):
        h = torch.relu(self.l2(torch.relu(self.l1(x))))
        return F.cross_entropy(self.l3(h), y)


class Emb(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(50, 16)
        self.l1 = nn.Linear(16, 16)
        self.l2 = nn.Linear(16, 50)

    def forward(self, ids):
        return self.l2(torch.relu(self.l1(self.emb(ids)))).mean(1)


class TiedEmb(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(50, 16)
        self.l1 = nn.Linear(16, 16)
        self.ln = nn.LayerNorm(16)

    def forward(self, ids, y):
        h = self.ln(torch.relu(self.l1(self.emb(ids))))
        logits = F.linear(h, self.emb.weight)
        return F.cross_entropy(logits.reshape(-1, 50), y.reshape(-1))


class LayerNormNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 32)
        self.ln = nn.LayerNorm(32)
        self.l2 = nn.Linear(32, 16)

    def forward(self, x):
        return self.l2(self.ln(F.gelu(self.l1(x))))


class Deep(nn.Module):
    def __init__(self, n=8):
        super().__init__()
        self.layers = nn.ModuleList([nn.Linear(16, 16) for _ in range(n)])

    def forward(self, x):
        for l in self.layers:
            x = torch.tanh(l(x))
        return x


class BNNet(nn.Module):
    """BatchNorm buffers (running statistics) are non-gradient state that must live with their stage."""

    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(1, 4, 3, padding=1)
        self.bn1 = nn.BatchNorm2d(4)
        self.c2 = nn.Conv2d(4, 4, 3, padding=1)
        self.bn2 = nn.BatchNorm2d(4)
        self.fc = nn.Linear(4, 3)

    def forward(self, x):
        x = F.relu(self.bn1(self.c1(x)))
        x = F.relu(self.bn2(self.c2(x)))
        return self.fc(x.mean((2, 3)))


class SmallParam(nn.Module):
    """Parameters far smaller than any alignment or bucket size (a 2-wide bottleneck and a scalar gain)."""

    def __init__(self):
        super().__init__()
        self.down = nn.Linear(16, 2)
        self.up = nn.Linear(2, 16)
        self.gain = nn.Parameter(torch.ones(()))

    def forward(self, x):
        return self.up(torch.tanh(self.down(x))) * self.gain


class ConstMul(nn.Module):
    """A plain tensor attribute (neither parameter nor buffer) that the tracer must lift as a constant."""

    def __init__(self):
        super().__init__()
        self.l = nn.Linear(16, 16)
        self.c = torch.linspace(-1.0, 1.0, 16)

    def forward(self, x):
        return self.l(x) * self.c + 0.5


class OneOp(nn.Module):
    """No parameters at all: nothing to place, nothing to reduce, gradients only flow to the input."""

    def forward(self, x):
        return torch.tanh(x) * 2.0


class Identity(nn.Module):
    def forward(self, x):
        return x


def _refine(x, layer, steps: int):
    for i in range(steps):
        x = x + torch.tanh(layer(x)) * (0.5 / (i + 1))
    return x


class FuncLoop(nn.Module):
    """A helper with a loop that reuses one layer: the unrolled body reads the same parameter at every trip."""

    def __init__(self):
        super().__init__()
        self.inp = nn.Linear(16, 16)
        self.body = nn.Linear(16, 16)

    def forward(self, x):
        return _refine(self.inp(x), self.body, 3)


class BufferRO(nn.Module):
    """A buffer that is only read (a fixed mask): it travels with the stage that uses it and is never reduced."""

    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 16)
        self.l2 = nn.Linear(16, 16)
        self.register_buffer("mask", (torch.arange(16) % 2).float())

    def forward(self, x):
        return self.l2(torch.relu(self.l1(x)) * self.mask)


class BufferRW(nn.Module):
    """A buffer the forward pass overwrites (an exponential average of the activations' scale)."""

    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 16)
        self.l2 = nn.Linear(16, 16)
        self.register_buffer("ema", torch.ones(16))

    def forward(self, x):
        h = torch.relu(self.l1(x))
        if self.training:
            self.ema.mul_(0.9).add_(h.detach().abs().mean(0), alpha=0.1)
        return self.l2(h / (1.0 + self.ema))


_MODELS = {"small_param": SmallParam, "const_mul": ConstMul, "one_op": OneOp, "identity": Identity,
           "func_loop": FuncLoop, "buffer_ro": BufferRO, "buffer_rw": BufferRW, "bn": BNNet, "basic": Basic, "forkjoin": ForkJoin, "shared_input": SharedInput, "shared_param": SharedParam,
           "loss": LossOut, "emb": Emb, "tied": TiedEmb, "layernorm": LayerNormNet, "deep": Deep}


def build(name):
    return _MODELS[name]()


def inputs(name, B, g):
    if name == "bn":
        return (torch.randn(B, 1, 8, 8, generator=g),)
    if name == "basic":
        return (torch.randn(B, 1, 16, 16, generator=g),)
    if name == "loss":
        return torch.randn(B, 16, generator=g), torch.randint(0, 5, (B,), generator=g)
    if name == "emb":
        return (torch.randint(0, 50, (B, 6), generator=g),)
    if name == "tied":
        return torch.randint(0, 50, (B, 6), generator=g), torch.randint(0, 50, (B, 6), generator=g)
    return (torch.randn(B, 16, generator=g),)
