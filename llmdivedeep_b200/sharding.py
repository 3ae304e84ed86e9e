"""How the DSA path is split over the GPUs of one box (one process per GPU).

Nothing in the reference is distributed; these rules come from the structure of the path:
  * prefill indexer + top-k: query rows are independent -> each rank takes whole chunks of
    query rows, dealt in serpentine order so that the causal cost (row t scans t+1 keys) balances;
    the keys are replicated; no exchange.
  * prefill sparse MLA: by rows (same chunks, no exchange before the output) or by heads
    (H/world heads per rank; needs every rank to hold all top-k indices).
  * decode: sequences are independent -> contiguous slices of the batch.
  * the only collective is the all-gather of the attention output.
The helpers are pure index arithmetic plus one torch.distributed call, so they run under
gloo on CPU as well as nccl on GPUs.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def row_chunks(n_rows: int, world: int, rank: int, chunk: int = 256) -> List[Tuple[int, int]]:
    """[start, end) query-row ranges of `rank`: chunks of `chunk` rows dealt in serpentine order
    (0..world-1, then world-1..0, ...), which evens out the linearly growing causal cost."""
    if not (0 <= rank < world) or chunk <= 0:
        raise ValueError("bad rank/world/chunk")
    n_chunks = (n_rows + chunk - 1) // chunk
    out = []
    for rnd in range((n_chunks + world - 1) // world):
        c = rnd * world + (rank if rnd % 2 == 0 else world - 1 - rank)
        if c < n_chunks:
            out.append((c * chunk, min(n_rows, (c + 1) * chunk)))
    return out


def round_robin_blocks(n_rows: int, world: int, rank: int, block: int = 256) -> List[Tuple[int, int]]:
    """[start, end) query-row ranges of `rank` when blocks of `block` rows are dealt round-robin
    (block b -> rank b % world).  One round of `world` consecutive blocks is one all-gather that lands
    in row order in the full output, so no re-ordering pass is needed afterwards; the causal cost of the
    ranks differs by about 2 / rounds (rank world-1 always holds the latest block of a round)."""
    if not (0 <= rank < world) or block <= 0:
        raise ValueError("bad rank/world/block")
    n_blocks = (n_rows + block - 1) // block
    return [(b * block, min(n_rows, (b + 1) * block)) for b in range(rank, n_blocks, world)]


def rows_of(chunks: List[Tuple[int, int]], device=None) -> torch.Tensor:
    """Row indices covered by a list of ranges, ascending."""
    if not chunks:
        return torch.empty(0, dtype=torch.long, device=device)
    return torch.cat([torch.arange(a, b, device=device) for a, b in chunks])


def causal_cost(chunks: List[Tuple[int, int]], first_pos: int = 0) -> int:
    """Keys scanned by the causal indexer for these rows (row t scans first_pos + t + 1 keys)."""
    return sum((b - a) * (2 * first_pos + a + b + 1) // 2 for a, b in chunks)


def head_range(n_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice of attention heads of `rank` (sizes differ by at most one)."""
    base, extra = divmod(n_heads, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def batch_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice of decode sequences of `rank`."""
    return head_range(batch, world, rank)


_PERM_CACHE = {}


def _all_gather_flat(gathered: torch.Tensor, buf: torch.Tensor, world: int, group=None) -> None:
    """gathered[r * n : (r + 1) * n] = rank r's buf (n = buf.shape[0]); one fused collective under nccl,
    the list form elsewhere (gloo on CPU)."""
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, buf, group=group)
    else:
        dist.all_gather(list(gathered.view((world,) + tuple(buf.shape)).unbind(0)), buf, group=group)


def _row_permutation(n_rows: int, world: int, chunk: int, pad: int, device) -> torch.Tensor:
    """For every output row, its position in the rank-major gathered buffer [world * pad]."""
    key = (n_rows, world, chunk, pad, str(device))
    if key not in _PERM_CACHE:
        perm = torch.empty(n_rows, dtype=torch.long)
        for r in range(world):
            rows = rows_of(row_chunks(n_rows, world, r, chunk))
            perm[rows] = r * pad + torch.arange(rows.numel())
        _PERM_CACHE[key] = perm.to(device)
    return _PERM_CACHE[key]


def all_gather_rows(local: torch.Tensor, n_rows: int, world: int, chunk: int = 256, group=None) -> torch.Tensor:
    """Assemble the full [n_rows, ...] output from per-rank row-chunk results (row sharding): one
    all-gather into a rank-major buffer (ranks padded to the largest row count) and one gather that
    puts the rows back in order."""
    counts = [sum(b - a for a, b in row_chunks(n_rows, world, r, chunk)) for r in range(world)]
    pad = max(counts)
    if local.shape[0] == pad:
        buf = local.contiguous()
    else:
        buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
        buf[: local.shape[0]] = local
    gathered = local.new_empty((world * pad,) + tuple(local.shape[1:]))
    _all_gather_flat(gathered, buf, world, group)
    return gathered.index_select(0, _row_permutation(n_rows, world, chunk, pad, local.device))


def all_gather_heads(local: torch.Tensor, n_heads: int, world: int, group=None) -> torch.Tensor:
    """Assemble [T, n_heads, D] from per-rank head slices [T, h_r, D] (head sharding)."""
    sizes = [head_range(n_heads, world, r) for r in range(world)]
    pad = max(b - a for a, b in sizes)
    if local.shape[1] == pad:
        buf = local.contiguous()
    else:
        buf = local.new_zeros((local.shape[0], pad, local.shape[2]))
        buf[:, : local.shape[1]] = local
    gathered = local.new_empty((world,) + tuple(buf.shape))
    _all_gather_flat(gathered.view((world * buf.shape[0],) + tuple(buf.shape[1:])), buf, world, group)
    if all(b - a == pad for a, b in sizes):
        return gathered.permute(1, 0, 2, 3).reshape(local.shape[0], n_heads, local.shape[2])
    return torch.cat([gathered[r][:, : b - a] for r, (a, b) in enumerate(sizes)], dim=1)


def all_gather_batch(local: torch.Tensor, batch: int, world: int, group=None) -> torch.Tensor:
    """Assemble [batch, ...] decode outputs from contiguous per-rank slices."""
    sizes = [batch_range(batch, world, r) for r in range(world)]
    pad = max(b - a for a, b in sizes)
    if local.shape[0] == pad:
        buf = local.contiguous()
    else:
        buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
        buf[: local.shape[0]] = local
    gathered = local.new_empty((world, pad) + tuple(local.shape[1:]))
    _all_gather_flat(gathered.view((world * pad,) + tuple(local.shape[1:])), buf, world, group)
    if all(b - a == pad for a, b in sizes):
        return gathered.reshape((batch,) + tuple(local.shape[1:]))
    return torch.cat([gathered[r][: b - a] for r, (a, b) in enumerate(sizes)], dim=0)


def all_gather_round(out_full: torch.Tensor, local_block: torch.Tensor, round_index: int, n_rows: int, world: int,
                     block: int = 256, group=None) -> None:
    """One round of the round-robin block split: every rank contributes its block of round
    `round_index` (rows [(round*world + rank)*block, ...)), and the `world` blocks land side by side, in
    row order, in out_full[round*world*block : (round+1)*world*block].  A full round is ONE collective
    straight into the output; the last, ragged round goes through a padded buffer."""
    lo = round_index * world * block
    hi = min(n_rows, lo + world * block)
    if hi - lo == world * block:
        _all_gather_flat(out_full[lo:hi], local_block, world, group)
        return
    buf = local_block.new_zeros((block,) + tuple(out_full.shape[1:]))
    buf[: local_block.shape[0]] = local_block
    gathered = local_block.new_empty((world * block,) + tuple(out_full.shape[1:]))
    _all_gather_flat(gathered, buf, world, group)
    out_full[lo:hi] = gathered[: hi - lo]
