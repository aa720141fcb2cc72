"""Shared builders for the GPU tests (inputs in the style of the reference's tests/utils.py:15-70)."""
import torch


def make_routing(num_tokens, num_topk, num_experts, seed, device, sentinel_p=0.0, empty_expert=None,
                 distinct=True):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if distinct:
        idx = torch.stack([torch.randperm(num_experts, generator=g)[:num_topk] for _ in range(num_tokens)]) \
            if num_tokens > 0 else torch.zeros(0, num_topk, dtype=torch.int64)
    else:
        idx = torch.randint(0, num_experts, (num_tokens, num_topk), generator=g)
    if sentinel_p > 0:
        idx = torch.where(torch.rand(num_tokens, num_topk, generator=g) < sentinel_p, torch.full_like(idx, -1), idx)
    if empty_expert is not None:
        idx = torch.where(idx == empty_expert, torch.full_like(idx, -1), idx)
    w = torch.rand(num_tokens, num_topk, generator=g, dtype=torch.float32)
    return idx.to(torch.int64).to(device), w.to(device)


def make_pool_case(num_experts, freqs, hidden, seed, device, tile_m=128, garbage_padding=False):
    """A hand-built pool: expert e has freqs[e] valid rows. Returns dict of tensors."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    tiles = [(f + tile_m - 1) // tile_m for f in freqs]
    off = [0]
    for t in tiles:
        off.append(off[-1] + t)
    total = off[-1]
    tkp = total * tile_m
    pool = torch.zeros(tkp, hidden)
    recv_token = torch.full((tkp,), -1, dtype=torch.int32)
    tile_e = torch.zeros(total, dtype=torch.int32)
    target = torch.zeros(total, dtype=torch.int32)
    nxt = 0
    for e, f in enumerate(freqs):
        r0 = off[e] * tile_m
        pool[r0:r0 + f] = torch.randn(f, hidden, generator=g)
        recv_token[r0:r0 + f] = torch.arange(nxt, nxt + f, dtype=torch.int32)
        nxt += f
        for j in range(tiles[e]):
            tile_e[off[e] + j] = e
            target[off[e] + j] = min(tile_m, f - j * tile_m)
    if garbage_padding:
        pad = recv_token < 0
        pool[pad] = float("inf")
    return dict(pool=pool.to(torch.bfloat16).to(device), recv_token=recv_token.to(device),
                tile_e=tile_e.to(device), target=target.to(device),
                offsets=torch.tensor(off, dtype=torch.int32, device=device),
                freqs=torch.tensor(freqs, dtype=torch.int32, device=device), total_tiles=total, tkp=tkp,
                num_valid=nxt)
