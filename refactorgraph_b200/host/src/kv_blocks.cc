#include "rg/kv_blocks.h"
#include <algorithm>

namespace refactor::runtime {

    KvBlockAllocator::KvBlockAllocator(uint32_t nBlocks, uint32_t pageSize, uint32_t maxSeqs, uint32_t maxBlocksPerSeq)
        : _nBlocks(nBlocks), _page(pageSize), _maxSeqs(maxSeqs), _maxBlocks(maxBlocksPerSeq),
          _table(static_cast<size_t>(maxSeqs) * maxBlocksPerSeq, -1), _rowUsed(maxSeqs, 0) {
        if (!nBlocks || !pageSize || !maxSeqs || !maxBlocksPerSeq) throw std::runtime_error("KvBlockAllocator: every size must be positive");
        _free.reserve(nBlocks);
        for (uint32_t b = nBlocks; b-- > 0;) _free.push_back(static_cast<int32_t>(b));// block 0 is handed out first
    }

    KvBlockAllocator::Seq const &KvBlockAllocator::find(int64_t id) const {
        auto it = _seqs.find(id);
        if (it == _seqs.end()) throw std::runtime_error("KvBlockAllocator: unknown sequence " + std::to_string(id));
        return it->second;
    }

    uint32_t KvBlockAllocator::addSequence(int64_t id, uint32_t tokens) {
        if (_seqs.count(id)) throw std::runtime_error("KvBlockAllocator: sequence " + std::to_string(id) + " already exists");
        const uint32_t need = (tokens + _page - 1) / _page;
        if (need > _maxBlocks) throw std::runtime_error("KvBlockAllocator: sequence longer than a table row can address");
        if (need > _free.size()) throw std::runtime_error("KvBlockAllocator: out of blocks");
        const auto rowIt = std::find(_rowUsed.begin(), _rowUsed.end(), 0);
        if (rowIt == _rowUsed.end()) throw std::runtime_error("KvBlockAllocator: no free table row");
        const uint32_t row = static_cast<uint32_t>(rowIt - _rowUsed.begin());
        *rowIt = 1;
        for (uint32_t j = 0; j < need; ++j) {
            _table[static_cast<size_t>(row) * _maxBlocks + j] = _free.back();
            _free.pop_back();
        }
        _seqs.emplace(id, Seq{row, tokens, need});
        return row;
    }

    uint32_t KvBlockAllocator::append(int64_t id, uint32_t n) {
        auto it = _seqs.find(id);
        if (it == _seqs.end()) throw std::runtime_error("KvBlockAllocator: unknown sequence " + std::to_string(id));
        Seq &s = it->second;
        const uint32_t need = (s.tokens + n + _page - 1) / _page;
        const uint32_t extra = need > s.blocks ? need - s.blocks : 0;
        if (need > _maxBlocks) throw std::runtime_error("KvBlockAllocator: sequence would outgrow its table row");
        if (extra > _free.size()) throw std::runtime_error("KvBlockAllocator: out of blocks");
        for (uint32_t j = s.blocks; j < need; ++j) {
            _table[static_cast<size_t>(s.row) * _maxBlocks + j] = _free.back();
            _free.pop_back();
        }
        s.blocks = need, s.tokens += n;
        return extra;
    }

    void KvBlockAllocator::release(int64_t id) {
        auto it = _seqs.find(id);
        if (it == _seqs.end()) throw std::runtime_error("KvBlockAllocator: unknown sequence " + std::to_string(id));
        Seq const &s = it->second;
        for (uint32_t j = s.blocks; j-- > 0;) {
            auto &slot = _table[static_cast<size_t>(s.row) * _maxBlocks + j];
            _free.push_back(slot);
            slot = -1;
        }
        _rowUsed[s.row] = 0;
        _seqs.erase(it);
    }

    uint32_t KvBlockAllocator::length(int64_t id) const { return find(id).tokens; }
    uint32_t KvBlockAllocator::row(int64_t id) const { return find(id).row; }
    std::vector<int32_t> KvBlockAllocator::blocks(int64_t id) const {
        Seq const &s = find(id);
        auto first = _table.begin() + static_cast<long>(static_cast<size_t>(s.row) * _maxBlocks);
        return std::vector<int32_t>(first, first + s.blocks);
    }
    std::vector<int64_t> KvBlockAllocator::lengths() const {
        std::vector<int64_t> ans(_maxSeqs, 0);
        for (auto const &[id, s] : _seqs) ans[s.row] = s.tokens;
        return ans;
    }

}// namespace refactor::runtime
