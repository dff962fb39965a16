"""Seeded synthetic EXL3 expert banks, activations and routing tables.

The reference is measured on private model weights and prompts that are not available; tensors with the
reference's shapes and the value distributions of the benchmark definition stand in for them:
  trellis words  uniform random 32-bit words                         [E1][K/16][N/16][32]
  scales         sign(+-1, p = 1/2) * U(0.5, 1.5) as fp16            suh_*[E1][K], svh_*[E1][N]
  activations    N(0, 1) rounded to bf16 (fp16 for the single-linear case)
  router         logits N(0,1) per (token, expert) [+ one per-batch bias vector]; scores = sigmoid(logits);
                 picks = top-k by score, ties to the lower id; weights = score / sum(scores);
                 a row is its top-k routed ids followed by the shared id E with weight 1.
All generators are numpy `Generator(PCG64(seed))`, so a seed gives the same tensors on every machine.
"""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16), the integer formula of the reference
    (src/experts.rs:19-21)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return (((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) & np.uint32(0xFFFF)).astype(
        np.uint16)


def bf16_bits_to_f32(h):
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def scales(g, n_experts, n, scale=1.0):
    sign = np.where(g.random((n_experts, n)) < 0.5, -1.0, 1.0)
    return (sign * g.uniform(0.5, 1.5, (n_experts, n)) * scale).astype(np.float16)


def expert_bank(seed, hidden=2048, inter=1536, experts=64, svh_scale=False):
    """The nine tensors of a bank of `experts` routed experts plus the shared expert (id `experts`).
    svh_scale=True divides svh_g / svh_u by 1.244 * sqrt(hidden) so that gate/up pre-activations have unit
    variance and the SwiGLU clamp does not saturate (the un-saturated parity variant)."""
    g = rng(seed)
    E1 = experts + 1
    words = lambda K, N: g.integers(0, 1 << 32, size=(E1, K // 16, N // 16, 32), dtype=np.uint64).astype(np.uint32)
    s = 1.0 / (1.244 * np.sqrt(hidden)) if svh_scale else 1.0
    sd = 1.0 / (1.244 * np.sqrt(inter)) if svh_scale else 1.0
    return {
        "gt": words(hidden, inter), "ut": words(hidden, inter), "dt": words(inter, hidden),
        "suh_g": scales(g, E1, hidden), "suh_u": scales(g, E1, hidden), "suh_d": scales(g, E1, inter),
        "svh_g": scales(g, E1, inter, s), "svh_u": scales(g, E1, inter, s), "svh_d": scales(g, E1, hidden, sd),
    }


def activations_bf16(seed, rows, hidden=2048):
    """N(0,1) activations as bf16 bit patterns, uint16 [rows][hidden]."""
    return f32_to_bf16_bits(rng(seed).standard_normal((rows, hidden)).astype(np.float32))


def route(seed, rows, experts=64, topk=4, shared_bias=False, uniform=False):
    """-> picks int32 [rows][topk+1], weights fp32 [rows][topk+1].
    shared_bias: add one N(0,1) bias vector to every token's logits (tokens then overlap on about half of
    their experts: the speculative-verify case).  uniform: `topk` distinct experts uniformly at random per
    token (the prefill case)."""
    g = rng(seed)
    if uniform:
        logits = g.random((rows, experts))
        scores = 1.0 / (1.0 + np.exp(-g.standard_normal((rows, experts))))
        order = np.argsort(-logits, axis=1, kind="stable")[:, :topk]
    else:
        logits = g.standard_normal((rows, experts))
        if shared_bias:
            logits = logits + g.standard_normal((1, experts))
        scores = 1.0 / (1.0 + np.exp(-logits))
        order = np.argsort(-scores, axis=1, kind="stable")[:, :topk]      # stable: ties go to the lower id
    top = np.take_along_axis(scores, order, axis=1)
    w = (top / top.sum(axis=1, keepdims=True)).astype(np.float32)
    picks = np.concatenate([order.astype(np.int32), np.full((rows, 1), experts, np.int32)], axis=1)
    weights = np.concatenate([w, np.ones((rows, 1), np.float32)], axis=1)
    return np.ascontiguousarray(picks), np.ascontiguousarray(weights)


def to_device(bank, device="cuda"):
    """numpy bank -> dict of torch CUDA tensors (uint32 words are carried as int32 bit patterns)."""
    import torch
    out = {}
    for k, v in bank.items():
        a = v.view(np.int32) if v.dtype == np.uint32 else v
        out[k] = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return out


def device_bank(seed, hidden=2048, inter=1536, experts=64, device="cuda"):
    """A bank generated directly on the GPU (torch generator): used for the 47-layer benchmark stack, where
    14 GB of random words would take minutes to draw on the host.  Same shapes and distributions."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    E1 = experts + 1

    def words(K, N):
        return torch.randint(-(1 << 31), (1 << 31) - 1, (E1, K // 16, N // 16, 32), dtype=torch.int32, device=device,
                             generator=g)

    def sc(n):
        sign = torch.where(torch.rand((E1, n), device=device, generator=g) < 0.5, -1.0, 1.0)
        return (sign * (0.5 + torch.rand((E1, n), device=device, generator=g))).to(torch.float16)

    return {"gt": words(hidden, inter), "ut": words(hidden, inter), "dt": words(inter, hidden),
            "suh_g": sc(hidden), "suh_u": sc(hidden), "suh_d": sc(inter),
            "svh_g": sc(inter), "svh_u": sc(inter), "svh_d": sc(hidden)}
