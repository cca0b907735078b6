// Peer-memory mailbox layout and the flag-in-data store / poll pair shared by the all-reduce kernel
// (tp.cu) and the matmul whose epilogue does the all-reduce itself (gemm.cu).
//
// A message of n 16-bit elements is n/4 units of four elements. A unit travels as one 16-byte
// store {lo32, epoch, hi32, epoch}: each 8-byte half carries its own flag, so a reader that sees
// the epoch in both halves has the data, with no fence and no separate flag write.
//
// Mailbox of one rank (written by its peers over NVLink, read locally):
//   [0, R)            two-shot: incoming partials of my slice, [sender][unit of slice]
//   [R, 2R)           two-shot: incoming results, [owner][unit of slice]
//   [2R, 2R + S)      one-shot, even epochs: incoming whole partials, [sender][unit of message]
//   [2R + S, 2R + 2S) one-shot, odd epochs
#pragma once
#include <stdint.h>

constexpr uint32_t P2P_MAX_ELEMS = 512 * 1024;                        // two-shot: 1 MiB of 16-bit elements
constexpr uint64_t P2P_REGION_BYTES = (uint64_t)P2P_MAX_ELEMS * 4;    // R: n/4 units x 16 bytes
constexpr uint64_t P2P_ONESHOT_BYTES = 8ull << 20;                    // S: world x (n/4) units x 16 bytes (64 x 4096 at 8 ranks)
constexpr uint64_t P2P_MAILBOX_BYTES = 2 * P2P_REGION_BYTES + 2 * P2P_ONESHOT_BYTES;
constexpr uint32_t P2P_WAIT_LIMIT = 1u << 22;                         // polls before a thread gives up

__device__ __forceinline__ uint64_t p2p_oneshot_offset(uint32_t epoch) {
    return 2 * P2P_REGION_BYTES + (uint64_t)(epoch & 1u) * P2P_ONESHOT_BYTES;
}
__device__ __forceinline__ void ll_store(uint8_t* base, uint64_t unit, uint2 d, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(base + unit * 16), "r"(d.x), "r"(epoch), "r"(d.y), "r"(epoch)
                 : "memory");
}
// Poll one unit until both halves carry `epoch`; false after `limit` polls (a peer that never sends: the
// caller records the failure and returns, the host reports it).
__device__ __forceinline__ bool ll_load(const uint8_t* base, uint64_t unit, uint32_t epoch, uint2* d, uint32_t limit = P2P_WAIT_LIMIT) {
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t a, fa, b, fb;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb) : "l"(base + unit * 16) : "memory");
        if (fa == epoch && fb == epoch) {
            *d = make_uint2(a, b);
            return true;
        }
        if (it > 1024) __nanosleep(100);
    }
    return false;
}
