"""Device-independent synthetic tensors for fixtures: integer hashing followed by
operations that are exact in fp32, so torch on the CPU and on CUDA give the same bits."""
import torch


def hash_uniform(count, seed, device="cpu", offset=0):
    """count values in [-1, 1), multiples of 2^-15."""
    i = torch.arange(offset, offset + count, dtype=torch.int64, device=device)
    x = (i * 2654435761 + (seed + 1) * 40503) & 0xFFFFFFFF
    x = x ^ (x >> 15)
    x = (x * 2246822519) & 0xFFFFFFFF
    x = x ^ (x >> 13)
    x = (x * 3266489917) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    return ((x & 0xFFFF).to(torch.float32) - 32768.0) * (1.0 / 32768.0)


def expert_weights_chunk(first_expert, experts, n_out, k_in, seed, device="cpu", scale=0.0346):
    """fp32 [experts, n_out, k_in], roughly uniform with std 0.02."""
    per = n_out * k_in
    flat = hash_uniform(experts * per, seed, device, offset=first_expert * per)
    return (flat * scale).view(experts, n_out, k_in)


def activations(tokens, width, seed, device="cpu", scale=1.7):
    """bf16 [tokens, width]: sum of two hashed uniforms, std about 1."""
    a = hash_uniform(tokens * width, seed, device)
    b = hash_uniform(tokens * width, seed + 1000003, device)
    return ((a + b) * scale).to(torch.bfloat16).view(tokens, width)
