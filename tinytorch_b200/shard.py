"""Multi-GPU partitioning of the attention path: contiguous batch x head ranges.

Attention units are independent: one (batch, kv head) pair together with the
query heads that share it.  Because tensors are dense [B, H, S, D]
(reference: src/Tensor/TensorImpl.cpp:13-31), a contiguous range of the
flattened B*Hkv index is one contiguous byte range of Q, K, V and O, so a rank's
shard is a plain view and no kernel needs a collective.  The only exchange is an
optional all-gather of O in head-parallel mode, with the semantics of the
reference's BackendNCCL::allGather (src/Distributed/BackendNCCL.cpp:49-62): rank
r's block lands at offset r of the gathered buffer.
"""
import torch
import torch.distributed as dist


def unit_range(n_units, rank, world):
    """Contiguous [begin, end) of `n_units` for `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, rem = divmod(n_units, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def balanced_ranges(weights, world):
    """Contiguous [begin, end) per rank with near-equal total weight (e.g. the valid cache rows of each unit
    in decode, where equal counts of units can differ by a third in work).  Ranges cover all units in order;
    a rank may get none.  Deterministic in (weights, world), so every rank computes the same list."""
    if world <= 0:
        raise ValueError("bad world")
    n = len(weights)
    total = float(sum(weights))
    bounds, acc, u = [0], 0.0, 0
    for r in range(1, world):
        target = total * r / world
        while u < n and acc + weights[u] / 2.0 <= target:  # a unit goes to the side its middle falls on
            acc += weights[u]
            u += 1
        bounds.append(u)
    bounds.append(n)
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def shard_bh(t, n_kv_units, rank, world):
    """View of the rank's units of a dense [B, H, S, D] tensor as [1, units*g, S, D].

    `n_kv_units` = B * Hkv; H may be Hq (= g * Hkv) or Hkv.
    """
    B, H, S, D = t.shape
    if not t.is_contiguous():
        raise ValueError("sharding needs the dense layout")
    g = (B * H) // n_kv_units
    b0, b1 = unit_range(n_kv_units, rank, world)
    return t.view(B * H, S, D)[b0 * g:b1 * g].unsqueeze(0)


def all_gather_output(o_local, n_kv_units, world, group=None, group_size=None, ranges=None):
    """Gather per-rank O shards ([1, units_r*g, L, D]) into [sum units*g, L, D].

    Uses all_gather on equal-sized padded blocks when shard sizes differ.  `group_size` is g, the number of
    query heads per kv head; when it is not given it is taken from the largest local shard over the ranks
    (a rank without units cannot tell from its own, empty shard).  `ranges`: the per-rank unit ranges when
    they are not the equal-count ones of unit_range (see balanced_ranges).
    """
    sizes = list(ranges) if ranges is not None else [unit_range(n_kv_units, r, world) for r in range(world)]
    if len(sizes) != world or sizes[0][0] != 0 or sizes[-1][1] != n_kv_units:
        raise ValueError("ranges must cover the units in rank order")
    mine = sizes[dist.get_rank(group)]
    if group_size is None:
        units = mine[1] - mine[0]
        gt = torch.tensor([o_local.shape[1] // units if units else 0], dtype=torch.int64, device=o_local.device)
        dist.all_reduce(gt, op=dist.ReduceOp.MAX, group=group)
        group_size = int(gt.item())
    g = group_size
    if o_local.shape[1] != (mine[1] - mine[0]) * g:
        raise ValueError("local shard has %d rows of heads, expected %d" % (o_local.shape[1], (mine[1] - mine[0]) * g))
    mx = max(e - b for b, e in sizes) * g
    pad = torch.zeros((mx,) + tuple(o_local.shape[2:]), dtype=o_local.dtype, device=o_local.device)
    pad[:o_local.shape[1]] = o_local[0]
    outs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(outs, pad, group=group)
    return torch.cat([outs[r][:(e - b) * g] for r, (b, e) in enumerate(sizes)], dim=0)
