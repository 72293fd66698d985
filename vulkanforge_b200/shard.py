"""Multi-GPU partitioning of the KV-cache hot path (one process per GPU).

VulkanForge itself is single-GPU and single-sequence (``docs/BENCHMARKS.md``: "VulkanForge is
single-stream"; one ``current_seq_len`` in ``src/backend/vulkan/kv_cache.rs:208``), so nothing
here has a counterpart in it.  The path shards in two ways:

* by sequence -- every sequence lives wholly on one GPU; no communication on the data path
  (``assign_sequences``);
* by position -- one long sequence is cut into pages that are dealt round-robin to the GPUs
  (``PositionShards``).  Each GPU attends over the pages it holds and produces, per q-head, the
  softmax partial (max m, sum l, unnormalised output o).  One all-gather of those partials
  (``Hq * (D + 2)`` floats per GPU) followed by the log-sum-exp merge of
  ``vk_shaders/flash_attn_reduce.comp:51-80`` gives the full result on every GPU.

The exchange is either ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) followed by
``vfkv_merge_partials_packed``, or -- ``ShardedSequenceDecoder(exchange=...)`` -- peer stores issued
by the attention kernel itself into every GPU's ``PeerExchange`` buffer and a merge kernel that
waits, with a time limit, on arrival flags (``vfkv_attend_exchange``); the second form has no
library call on the data path and can be replayed from a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence


def assign_sequences(lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Longest-first greedy balancing of sequences over ranks by total context length.
    Returns, per rank, the indices of the sequences it owns."""
    loads = [0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i)):
        r = min(range(world_size), key=lambda r: (loads[r], r))
        owned[r].append(i)
        loads[r] += int(lengths[i])
    for o in owned:
        o.sort()
    return owned


@dataclass(frozen=True)
class PositionShards:
    """Round-robin pages of ``page`` positions: global position p is held by rank
    ``(p // page) % world_size`` at local position ``((p // page) // world_size) * page + p % page``.
    Appends therefore rotate over the GPUs instead of always landing on the last one, and every
    rank's share of a context of any length differs by at most one page."""
    world_size: int
    page: int = 256

    def owner(self, pos: int) -> int:
        return (pos // self.page) % self.world_size

    def local_pos(self, pos: int) -> int:
        return ((pos // self.page) // self.world_size) * self.page + pos % self.page

    def local_len(self, seq_len: int, rank: int) -> int:
        """How many of the positions [0, seq_len) rank holds (they occupy local [0, local_len))."""
        full_pages, rest = divmod(seq_len, self.page)
        n = (full_pages // self.world_size) * self.page
        extra = full_pages % self.world_size
        if rank < extra:
            n += self.page
        elif rank == extra:
            n += rest
        return n

    def local_capacity(self, max_seq_len: int) -> int:
        """Rows a rank's slab needs for contexts up to max_seq_len."""
        pages = (max_seq_len + self.page - 1) // self.page
        return ((pages + self.world_size - 1) // self.world_size) * self.page

    def global_positions(self, seq_len: int, rank: int) -> List[int]:
        """The global positions behind local 0 .. local_len-1, in local order."""
        out = []
        for page_id in range(rank, (seq_len + self.page - 1) // self.page, self.world_size):
            lo = page_id * self.page
            out.extend(range(lo, min(lo + self.page, seq_len)))
        return out


def packed_partial_floats(n_q_heads: int, head_dim: int) -> int:
    """Floats one rank contributes: m[Hq], l[Hq], o[Hq][D]."""
    return n_q_heads * (head_dim + 2)


def all_gather_partials(local_packed, group=None):
    """All-gathers every rank's packed partial (a 1-D float32 tensor) into a
    [world_size, packed_floats] tensor on the same device."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    n = local_packed.numel()
    out = torch.empty(world * n, dtype=local_packed.dtype, device=local_packed.device)
    dist.all_gather_into_tensor(out, local_packed.contiguous().view(-1), group=group)
    return out.view(world, n)


class ShardedSequenceDecoder:
    """Position-sharded decode attention for one long sequence on this rank's GPU.

    ``fwd`` is this rank's ``CudaForward`` over a cache whose ``max_seq_len`` is at least
    ``shards.local_capacity(global max)``; slot 0 holds this rank's pages.
    """

    def __init__(self, fwd, shards: PositionShards, rank: int, group=None, exchange=None):
        import torch
        self.fwd, self.shards, self.rank, self.group = fwd, shards, rank, group
        self.exchange = exchange      # a connected PeerExchange: partials travel by peer stores, no collective
        hd = fwd.kv_cache.config.head_dim
        self.n_rows, self.head_dim = fwd.n_heads, hd
        self.packed = torch.zeros(packed_partial_floats(fwd.n_heads, hd), dtype=torch.float32, device="cuda")

    def append(self, layer: int, k_src, v_src, position: int) -> bool:
        """Stores the token of global ``position`` if this rank owns its page; returns whether it did."""
        if self.shards.owner(position) != self.rank:
            return False
        self.fwd.step_kv_write(layer, k_src, v_src, self.shards.local_pos(position), 0)
        return True

    def prefill(self, layer: int, k_src, v_src, base_pos: int, n_tokens: int) -> int:
        """Chunked-prefill append: stores the rows of [base_pos, base_pos + n_tokens) this rank owns
        (one launch for the chunk; the kernel skips the other ranks' pages) and returns how many
        those are.  k_src / v_src are torch tensors [n_tokens][kv_heads][D]."""
        self.fwd.b_step_kv_write_sharded(layer, k_src, v_src, n_tokens, base_pos, self.shards.world_size,
                                         self.shards.page, self.rank)
        return self.shards.local_len(base_pos + n_tokens, self.rank) - self.shards.local_len(base_pos, self.rank)

    def decode(self, layer: int, q, k_src, v_src, out, position: int):
        """One decode step of global ``position``: append (owner rank only) and attention over
        [0, position], merged over the ranks.  With a peer exchange the owner's attention kernel
        stores the new row itself."""
        if self.exchange is None:
            self.append(layer, k_src, v_src, position)
            return self.attend(layer, q, out, position + 1)
        mine = self.shards.owner(position) == self.rank
        self.fwd.attend_exchange(self.exchange, layer, q, 0, self.shards.local_len(position + 1, self.rank), out,
                                 k_new=k_src if mine else None, v_new=v_src if mine else None)
        return out

    def attend(self, layer: int, q, out, seq_len: int):
        """Attention of one query token over global positions [0, seq_len): local partial, one
        all-gather, merge.  ``out`` [Hq][D] is complete on every rank."""
        n, hd = self.n_rows, self.head_dim
        if self.exchange is not None:
            self.fwd.attend_exchange(self.exchange, layer, q, 0, self.shards.local_len(seq_len, self.rank), out)
            return out
        m, l, o = self.packed[:n], self.packed[n:2 * n], self.packed[2 * n:]
        self.fwd.attend_partial(layer, q, 0, self.shards.local_len(seq_len, self.rank), m, l, o)
        gathered = all_gather_partials(self.packed, self.group)
        self.fwd.merge_partials_packed(gathered, gathered.shape[0], n, hd, out)
        return out
