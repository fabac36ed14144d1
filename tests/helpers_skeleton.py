"""A one-layer model skeleton with the member names the artifact metadata addresses
(`model.layers.<i>.<path>.weight`), used by the loader tests and by the script that
generates their fixture."""
import torch
import torch.nn as nn


class Qwen3_5MLP(nn.Module):      # the class name the reference's MLP fusion pass looks for
    def __init__(self, hidden, inter):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)
        self.act_fn = nn.SiLU()

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class _Norm(nn.Module):
    def __init__(self, n):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(n))       # zero-centered gain: 1 + w


class _Attn(nn.Module):
    def __init__(self, hidden):
        super().__init__()
        self.in_proj_qkv = nn.Linear(hidden, 3 * hidden, bias=True)


class _Layer(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.linear_attn = _Attn(hidden)
        self.post_attention_layernorm = _Norm(hidden)
        self.mlp = Qwen3_5MLP(hidden, inter)


class _Text(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.layers = nn.ModuleList([_Layer(hidden, inter)])


class _Wrapper(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.model = _Text(hidden, inter)


def tiny_skeleton(hidden: int = 128, inter: int = 256, seed: int = 7) -> nn.Module:
    torch.manual_seed(seed)
    m = _Wrapper(hidden, inter)
    with torch.no_grad():
        m.model.layers[0].linear_attn.in_proj_qkv.bias.copy_(
            0.1 * torch.randn(3 * hidden, generator=torch.Generator().manual_seed(seed)))
    return m


def tiny_skeleton_with_heads(hidden: int = 128, inter: int = 256, vocab: int = 256,
                             seed: int = 7) -> nn.Module:
    """The same skeleton plus the two head modules the head artifacts address:
    `lm_head` on the wrapper and `embed_tokens` on the text model."""
    m = tiny_skeleton(hidden, inter, seed)
    m.lm_head = nn.Linear(hidden, vocab, bias=False)
    m.model.embed_tokens = nn.Embedding(vocab, hidden)
    return m
