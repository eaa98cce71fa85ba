"""Host-side shard planning for the Hyena block: channel shards for prefill, batch shards for decode.

Every Hyena operator is independent per (batch element, hidden channel) along the whole sequence, so a shard
of channels (whole filter groups, whole q/k/v triplets) or of batch elements is computed without any exchange.
The only collective sits at the boundary the model already has: gathering the block output ``y [B, L, D/W]``
of the W ranks before the (replicated) output projection.  The reference has no counterpart: it places whole
layers on GPUs (``vortex/model/model.py:650-671``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch


def channel_range(D: int, G: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous hidden channels [d0, d1) of `rank`: whole filter groups, as even as possible."""
    if D % G:
        raise ValueError("D must be a multiple of the number of filter groups")
    if world > G:
        raise ValueError(f"cannot cut {G} filter groups into {world} shards")
    per, g_lo = D // G, (G * rank) // world
    g_hi = (G * (rank + 1)) // world
    return g_lo * per, g_hi * per


def batch_range(B: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous batch elements [b0, b1) of `rank` (decode: all caches are per sample)."""
    return (B * rank) // world, (B * (rank + 1)) // world


def packed_columns(D: int, d0: int, d1: int, layout: str, num_heads: int = 1) -> torch.Tensor:
    """Indices of the packed projection columns (of 3D) that hold q, k, v of hidden channels [d0, d1),
    in the order of the shard's own packed tensor (same layout, D replaced by d1 - d0)."""
    d = torch.arange(d0, d1)
    if layout == "interleaved":
        return torch.stack([3 * d, 3 * d + 1, 3 * d + 2], dim=1).reshape(-1)
    if layout == "split":
        return torch.cat([d, D + d, 2 * D + d])
    if layout == "column_split":
        hd = D // num_heads
        if d0 % hd or d1 % hd:
            raise ValueError("column-split shards must hold whole heads")
        n, j = d // hd, d % hd
        base = n * 3 * hd + j
        return torch.stack([base.reshape(-1, hd), (base + hd).reshape(-1, hd), (base + 2 * hd).reshape(-1, hd)],
                           dim=1).reshape(-1)
    raise ValueError(f"unknown q/k/v layout {layout!r}")


def shard_block(params: Dict[str, Optional[torch.Tensor]], D: int, G: int, world: int, rank: int,
                layout: str = "interleaved", num_heads: int = 1) -> Dict[str, Optional[torch.Tensor]]:
    """Slice the inputs and parameters of one Hyena block for `rank`.

    params: u [B, L, 3D], w3 [3D, 1, 3], optional b3 [3D], h [G, 1, K] or modal log_poles / residues (/ theta /
    res_im) [G, S(,1)], Dp [D] or None.  Returns the same keys for a block of d1 - d0 channels."""
    d0, d1 = channel_range(D, G, world, rank)
    cols = packed_columns(D, d0, d1, layout, num_heads)
    g0, g1 = d0 // (D // G), d1 // (D // G)
    out: Dict[str, Optional[torch.Tensor]] = {}
    for key, t in params.items():
        if t is None:
            out[key] = None
        elif key == "u":
            if layout == "interleaved":          # contiguous run of columns: a view, no copy
                out[key] = t[..., 3 * d0:3 * d1]
            else:
                out[key] = t.index_select(-1, cols.to(t.device))
        elif key in ("w3", "b3"):
            out[key] = t.index_select(0, cols.to(t.device))
        elif key in ("h", "log_poles", "residues", "theta", "res_im"):
            out[key] = t[g0:g1]
        elif key == "Dp":
            out[key] = t[d0:d1]
        else:
            out[key] = t
    return out


def gather_channels(y_shard: torch.Tensor, group=None, widths=None, out: Optional[torch.Tensor] = None,
                    concat: bool = True) -> torch.Tensor:
    """All-gather the block outputs [B, L, D_r] of all ranks along the channel axis (the one collective at the
    shard boundary; NCCL over NVLink on GPUs, gloo in the CPU tests).

    ``widths``: the channel counts D_r of all ranks, e.g. from ``channel_range``; when omitted they are
    exchanged first (a small collective plus a host read).  Unequal shards (``channel_range`` hands out whole filter
    groups, so G % world != 0 gives shards that differ by one group) are padded to the widest shard for the
    exchange and cut back afterwards -- a collective with mismatched sizes across ranks is undefined on NCCL.
    ``out``: optional [world, B, L, D_max] receive buffer to reuse.  ``concat=False`` returns that rank-major
    buffer as it arrived (no further copy; a replicated projection can contract it block by block, and only
    ``[r, ..., :widths[r]]`` of each block is meaningful); the default concatenates to [B, L, D]."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return y_shard if concat else y_shard[None]
    if widths is None:
        mine = torch.tensor([y_shard.shape[-1]], dtype=torch.int64, device=y_shard.device)
        allw = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allw, mine, group=group)
        widths = [int(w.item()) for w in allw]
    widths = [int(w) for w in widths]
    if len(widths) != world or widths[dist.get_rank(group)] != y_shard.shape[-1]:
        raise ValueError(f"widths {widths} do not describe this group (this rank holds {y_shard.shape[-1]} channels)")
    wmax = max(widths)
    send = y_shard.contiguous()
    if send.shape[-1] != wmax:
        send = torch.nn.functional.pad(send, (0, wmax - send.shape[-1]))
    shape = (world,) + tuple(send.shape)
    if out is None:
        out = torch.empty(shape, device=send.device, dtype=send.dtype)
    elif tuple(out.shape) != shape or out.dtype != send.dtype or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {shape} tensor of the shard's dtype")
    # (the receive buffer is handed over in its "concatenated along dim 0" form, which every backend accepts)
    dist.all_gather_into_tensor(out.view((world * send.shape[0],) + tuple(send.shape[1:])), send, group=group)
    if not concat:
        return out
    return torch.cat([out[r, ..., :widths[r]] for r in range(world)], dim=-1)
