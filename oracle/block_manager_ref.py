"""Oracle (test infrastructure): Python restatement of the reference's paged-KV
bookkeeping — BlockAllocator / BlockManager (src/scheduler/block_manager.rs),
PrefixCache and hash_block (src/scheduler/prefix_cache.rs) and the Sequence block
arithmetic (src/scheduler/sequence.rs:80-92)."""
from __future__ import annotations

from collections import OrderedDict, deque

BLOCK_SIZE = 16            # block_manager.rs:25
PREFIX_CACHE_CAPACITY = 128  # block_manager.rs:115
MASK64 = (1 << 64) - 1


def hash_block(tokens) -> int:
    """FNV-1a over whole u32 tokens: xor then multiply (prefix_cache.rs:40-50)."""
    h = 0xCBF29CE484222325
    for t in tokens:
        h ^= int(t)
        h = (h * 0x100000001B3) & MASK64
    return h


def num_logical_blocks(length: int, block_size: int = BLOCK_SIZE) -> int:
    """len.div_ceil(block_size) (sequence.rs:80-82)."""
    return -(-length // block_size)


def last_block_num_filled(length: int, block_size: int = BLOCK_SIZE) -> int:
    """sequence.rs:85-92."""
    rem = length % block_size
    return block_size if (rem == 0 and length != 0) else rem


class BlockAllocator:
    """block_manager.rs:46-102: free list 0..n, allocate = pop_front, free = push_back
    when the refcount reaches zero."""

    def __init__(self, num_blocks: int):
        self.free_blocks = deque(range(num_blocks))
        self.allocated: dict[int, int] = {}

    def allocate(self):
        if not self.free_blocks:
            return None
        i = self.free_blocks.popleft()
        self.allocated[i] = 1
        return i

    def free(self, block_id: int) -> None:
        if block_id in self.allocated:
            self.allocated[block_id] -= 1
            if self.allocated[block_id] == 0:
                del self.allocated[block_id]
                self.free_blocks.append(block_id)

    def num_free(self) -> int:
        return len(self.free_blocks)

    def ref_count(self, block_id: int) -> int:
        return self.allocated.get(block_id, 0)

    def increment_ref(self, block_id: int) -> None:
        if block_id in self.allocated:
            self.allocated[block_id] += 1


class PrefixCache:
    """prefix_cache.rs:53-131 (FIFO eviction)."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.entries: dict[int, int] = {}
        self.order: deque[int] = deque()
        self.block_to_hash: dict[int, int] = {}

    def lookup(self, h: int):
        return self.entries.get(h)

    def insert(self, h: int, block_id: int) -> None:
        if h in self.entries:
            old = self.entries[h]
            if old != block_id:
                self.block_to_hash.pop(old, None)
            self.entries[h] = block_id
            self.block_to_hash[block_id] = h
            return
        if len(self.entries) >= self.capacity and self.order:
            victim = self.order.popleft()
            if victim in self.entries:
                vid = self.entries.pop(victim)
                self.block_to_hash.pop(vid, None)
        self.entries[h] = block_id
        self.order.append(h)
        self.block_to_hash[block_id] = h

    def remove_by_block_id(self, block_id: int) -> None:
        h = self.block_to_hash.pop(block_id, None)
        if h is not None:
            self.entries.pop(h, None)

    def __len__(self) -> int:
        return len(self.entries)


class BlockManager:
    """block_manager.rs:143-414 for single-sequence groups."""

    def __init__(self, num_gpu_blocks: int, num_cpu_blocks: int):
        self.block_size = BLOCK_SIZE
        self.gpu = BlockAllocator(num_gpu_blocks)
        self.cpu = BlockAllocator(num_cpu_blocks)
        self.block_tables: dict[int, list[int]] = {}
        self.prefix_cache = PrefixCache(PREFIX_CACHE_CAPACITY)
        self.block_hashes: dict[int, int] = {}

    def num_free_gpu_blocks(self) -> int:
        return self.gpu.num_free()

    def num_free_cpu_blocks(self) -> int:
        return self.cpu.num_free()

    def num_prefix_cached_blocks(self) -> int:
        return len(self.prefix_cache)

    def can_allocate(self, total_len: int) -> bool:
        return num_logical_blocks(total_len) <= self.gpu.num_free()

    def allocate(self, seq_id: int, prompt_ids, output_len: int = 0) -> int:
        """block_manager.rs:194-253; returns hit_blocks."""
        needed = num_logical_blocks(len(prompt_ids) + output_len)
        if needed > self.gpu.num_free() + len(self.prefix_cache):
            raise RuntimeError(f"not enough GPU blocks: need {needed}")
        table: list[int] = []
        hits = 0
        complete = len(prompt_ids) // self.block_size
        for b in range(complete):
            h = hash_block(prompt_ids[b * self.block_size:(b + 1) * self.block_size])
            cached = self.prefix_cache.lookup(h)
            if cached is not None:
                self.gpu.increment_ref(cached)
                table.append(cached)
                hits += 1
            else:
                i = self.gpu.allocate()
                if i is None:
                    raise RuntimeError("no free GPU blocks for allocation")
                table.append(i)
                self.block_hashes[i] = h
        for _ in range(needed - complete):
            i = self.gpu.allocate()
            if i is None:
                raise RuntimeError("no free GPU blocks for allocation")
            table.append(i)
        self.block_tables[seq_id] = table
        return hits

    def free(self, seq_id: int) -> None:
        """block_manager.rs:264-276."""
        table = self.block_tables.pop(seq_id, None)
        if table is None:
            return
        for block_id in table:
            if block_id in self.block_hashes:
                self.prefix_cache.insert(self.block_hashes[block_id], block_id)
            self.gpu.free(block_id)

    def can_append_slot(self, seq_id: int, total_len: int) -> bool:
        """block_manager.rs:284-308."""
        table = self.block_tables.get(seq_id)
        if table is None:
            return False
        if last_block_num_filled(total_len) == self.block_size and self.gpu.num_free() == 0:
            return False
        if table and self.gpu.ref_count(table[-1]) > 1 and self.gpu.num_free() == 0:
            return False
        return True

    def append_slot(self, seq_id: int, total_len: int):
        """block_manager.rs:314-351; returns the copy-on-write pairs."""
        cow = []
        table = self.block_tables[seq_id]
        filled = last_block_num_filled(total_len)
        if filled == self.block_size or not table:
            i = self.gpu.allocate()
            if i is None:
                raise RuntimeError("no free GPU blocks for append")
            table.append(i)
        else:
            last = table[-1]
            if self.gpu.ref_count(last) > 1:
                i = self.gpu.allocate()
                if i is None:
                    raise RuntimeError("no free GPU blocks for CoW")
                self.gpu.free(last)
                table[-1] = i
                cow.append((last, i))
        return cow

    def swap_out(self, seq_id: int):
        """block_manager.rs:359-380."""
        pairs = []
        table = self.block_tables[seq_id]
        for idx, gpu_id in enumerate(table):
            cpu_id = self.cpu.allocate()
            if cpu_id is None:
                raise RuntimeError("no free CPU blocks for swap_out")
            pairs.append((gpu_id, cpu_id))
            self.gpu.free(gpu_id)
            table[idx] = cpu_id
        return pairs

    def swap_in(self, seq_id: int):
        """block_manager.rs:385-406."""
        pairs = []
        table = self.block_tables[seq_id]
        for idx, cpu_id in enumerate(table):
            gpu_id = self.gpu.allocate()
            if gpu_id is None:
                raise RuntimeError("no free GPU blocks for swap_in")
            pairs.append((cpu_id, gpu_id))
            self.cpu.free(cpu_id)
            table[idx] = gpu_id
        return pairs

    def get_block_table(self, seq_id: int):
        return self.block_tables.get(seq_id)
