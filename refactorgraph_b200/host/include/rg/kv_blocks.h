// Block allocator for the paged KV cache: hands out the fixed-size blocks of a cache tensor
// [n_blocks, kv_heads, page, head_dim] to sequences and maintains the int32 block table [max_seqs, max_blocks_per_seq]
// that the paged kernels read (rg_kv_layout in include/rg_b200.h).
//
// It takes the place the reference gives to its device memory pool — MemPool over OffsetCalculator's best-fit free list
// (src/02hardware/src/mem_pool.cc, src/02hardware/src/mem_offset_calculator.cc:29-115), which the Nvidia device sizes at
// 90 % of free memory (src/02hardware/src/devices/nvidia/device.cc:24-35).  A KV cache needs neither best fit nor
// coalescing: every request is one block, so a LIFO free list is exact and O(1), and the cache tensor is allocated once
// by the caller at the size it chooses instead of by a grab of whatever is free on a shared GPU.
// Host-side only; not thread-safe (one serving loop owns it, like the reference's single-threaded Stream).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace refactor::runtime {

    class KvBlockAllocator {
    public:
        KvBlockAllocator(uint32_t nBlocks, uint32_t pageSize, uint32_t maxSeqs, uint32_t maxBlocksPerSeq);

        // Registers a sequence of `tokens` cached tokens in a free row of the table; returns the row.  Throws when no row or not
        // enough blocks are free (nothing is changed in that case).
        uint32_t addSequence(int64_t id, uint32_t tokens);
        // Makes room for `n` more tokens of a sequence (a new block each time a page boundary is crossed); returns the number of
        // blocks added.  Throws std::runtime_error when the free list or the table row runs out; the sequence is left unchanged.
        uint32_t append(int64_t id, uint32_t n = 1);
        // Returns a finished sequence's blocks to the free list and frees its row.
        void release(int64_t id);

        uint32_t freeBlocks() const { return static_cast<uint32_t>(_free.size()); }
        uint32_t length(int64_t id) const;
        uint32_t row(int64_t id) const;
        std::vector<int32_t> blocks(int64_t id) const;
        // the table as the kernels read it: row-major [max_seqs, max_blocks_per_seq]; unused entries are -1 (the kernels reject
        // negative block numbers instead of reading through them)
        std::vector<int32_t> const &table() const { return _table; }
        // cached tokens per table row (0 for free rows): the `lens` / `pos` state of a decode step
        std::vector<int64_t> lengths() const;
        uint32_t pageSize() const { return _page; }
        uint32_t maxSeqs() const { return _maxSeqs; }
        uint32_t maxBlocksPerSeq() const { return _maxBlocks; }
        uint32_t nBlocks() const { return _nBlocks; }

    private:
        struct Seq {
            uint32_t row, tokens, blocks;
        };
        Seq const &find(int64_t id) const;
        uint32_t _nBlocks, _page, _maxSeqs, _maxBlocks;
        std::vector<int32_t> _free;// LIFO
        std::vector<int32_t> _table;
        std::vector<char> _rowUsed;
        std::unordered_map<int64_t, Seq> _seqs;
    };

}// namespace refactor::runtime
