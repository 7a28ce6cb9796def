// Layout of a communicator's symmetric allocation (all_reduce.cu), shared with the kernels that write all-reduce input straight
// from their epilogue: header | slots A [2 parities][world source ranks] | slots B [2 parities].  A slot holds `capacity` data
// bytes as 32-byte lines: every 16-byte chunk travels as four {32-bit data, 32-bit flag} pairs.
#pragma once
#include "common.cuh"
namespace rg {
constexpr int AR_MAX_RANKS = 8;
constexpr size_t AR_HEADER_BYTES = 4096;
struct ArHeader {
    unsigned long long seq;// number of the call in flight (starts at 1)
    unsigned int done;     // CTAs of the current call that have read seq
    int status;            // 0 ok; 1 = a wait on a peer flag expired
};
// byte offset of the slot that holds rank `src`'s input of a call with parity q, inside any rank's allocation
__host__ __device__ __forceinline__ size_t ar_slot_offset(size_t capacity, int world, unsigned q, int src) {
    return AR_HEADER_BYTES + (static_cast<size_t>(q) * world + src) * (2 * capacity);
}
// Flag of call number seq: never 0 (slots start zeroed, so memory no call has written can never look complete) and
// different from the flag two calls earlier, which is what a slot of the same parity may still hold.
__host__ __device__ __forceinline__ uint32_t ar_flag(unsigned long long seq) { return static_cast<uint32_t>(seq % 0xffffffffull) + 1u; }
// What a kernel needs to write into the slots: filled by the host from a communicator
struct ArPeers {
    uint8_t *mine;
    uint8_t *peer[AR_MAX_RANKS];// peer[rank] = mine
    uint64_t capacity;
    int world, rank;
    int two_shot;// every rank must use the same variant for a call
};
}// namespace rg
