"""Tensor/pipeline/expert-parallel layout arithmetic.

Same split semantics as the reference so that a TP=N run of this engine shards every
tensor exactly where the reference would (``src/utils/split_util.h:8-99``):

* `task_range(N, splits, idx)` — even split when ``N % (splits*64) == 0``; otherwise the
  coarsest granularity of 64/16/2 that divides N, with the remainder going to low ranks
  (FFN 11008 over 8 ranks -> 4x1408 + 4x1344; 688 over 2 -> 352 + 336).
* `head_range(q, kv, splits, idx)` — contiguous query-head range and the covering KV range.
* PP stage layer ranges (``src/layers/decoder_block.h:33-40``) and the MoE slice rotation
  (``src/layers/mlp_llama.h:70-79``).  Expert-parallel placement is new (the reference
  only slices experts).
"""
from __future__ import annotations

from typing import List, Tuple


def task_range(n: int, splits: int, idx: int) -> Tuple[int, int]:
    if splits <= 0 or not (0 <= idx < splits):
        raise ValueError(f"bad split {idx}/{splits}")
    if n % (splits * 64) == 0:
        per = n // splits
        return idx * per, (idx + 1) * per
    gran = 1
    for cand in (64, 16, 2):
        if n % cand == 0:
            n //= cand
            gran = cand
            break
    base, rem = divmod(n, splits)
    if idx < rem:
        start = idx * (base + 1)
        end = start + base + 1
    else:
        start = (base + 1) * rem + (idx - rem) * base
        end = start + base
    return start * gran, end * gran


def task_range_gran(n: int, gran: int, splits: int, idx: int) -> Tuple[int, int]:
    if n % gran:
        raise ValueError(f"N ({n}) need to be multiple of granularity ({gran}).")
    s, e = task_range(n // gran, splits, idx)
    return s * gran, e * gran


def head_range(q_heads: int, kv_heads: int, splits: int, idx: int):
    """-> ((q_start, q_end), (kv_start, kv_end)); kv range covers the q range (GQA)."""
    base, rem = divmod(q_heads, splits)
    if idx < rem:
        start = idx * (base + 1)
        end = start + base + 1
    else:
        start = (base + 1) * rem + (idx - rem) * base
        end = start + base
    expand = q_heads // kv_heads if kv_heads > 0 else 1
    kv_start = start // expand
    kv_end = (end - 1) // expand + 1 if end > start else kv_start
    return (start, end), (kv_start, kv_end)


def vocab_range(vocab: int, splits: int, idx: int) -> Tuple[int, int]:
    """lm_head row split (``src/layers/dist_linear.h:49-64``)."""
    return task_range(vocab, splits, idx)


def pp_layer_range(num_layers: int, pp_size: int, pp_rank: int) -> Tuple[int, int]:
    """Layers of one pipeline stage; the reference requires divisibility, here the
    remainder goes to the first stages."""
    base, rem = divmod(num_layers, pp_size)
    start = pp_rank * base + min(pp_rank, rem)
    return start, start + base + (1 if pp_rank < rem else 0)


def moe_slice_index(tp_rank: int, tp_size: int, layer_id: int, expert_id: int, balance_dim: int = 0) -> int:
    """Rotated TP slice index for MoE experts so that uneven slices even out across
    layers (balance_dim 0) or experts (1) — ``XFT_MOE_SPLIT_BALANCE_DIM``."""
    rot = layer_id if balance_dim == 0 else expert_id
    return (tp_rank + rot) % tp_size


def expert_range(num_experts: int, ep_size: int, ep_rank: int) -> Tuple[int, int]:
    """Contiguous block of experts owned by an EP rank."""
    base, rem = divmod(num_experts, ep_size)
    start = ep_rank * base + min(ep_rank, rem)
    return start, start + base + (1 if ep_rank < rem else 0)


def expert_owner(expert_id: int, num_experts: int, ep_size: int) -> int:
    base, rem = divmod(num_experts, ep_size)
    cut = rem * (base + 1)
    if expert_id < cut:
        return expert_id // (base + 1)
    return rem + (expert_id - cut) // max(base, 1)


def block_owner(block: int, world: int) -> int:
    """Rank that reduces token block `block` in the fused prefill GEMM + all-reduce (round-robin)."""
    return block % world


def block_visit_order(num_blocks: int, world: int, rank: int, lag: int = -1) -> List[int]:
    """Order in which one rank's persistent CTAs visit the token blocks of a fused prefill GEMM + all-reduce.

    All ranks walk the blocks in index order, but a rank reaches a block it OWNS `lag` steps late (default: one round
    of `world` blocks): by then the other ranks, which pass that block at its natural position, have normally
    delivered their partial sums, so the owner's reduction does not wait.  Every rank's list is a permutation of
    ``range(num_blocks)``.  Liveness: give block j the key j on the ranks that do not own it and j + lag + 1/2 on its
    owner; each rank visits in key order, a wait at key j + lag + 1/2 depends on work at key j, and a CTA that is stuck
    earlier in its list is stuck at a smaller key, so every chain of waits runs down the keys and ends."""
    if lag < 0:
        lag = world
    out: List[int] = []
    for k in range(num_blocks + lag):
        if k < num_blocks and block_owner(k, world) != rank:
            out.append(k)
        if k >= lag and block_owner(k - lag, world) == rank:
            out.append(k - lag)
    return out
