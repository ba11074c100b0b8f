// gather.cuh - device role that stages a range of the sharded parameter space into local memory.
//
// ZeRO-3 layout: the flat bf16 parameter space [0, n_flat) is cut into `size` contiguous shards of
// n_shard elements, member r keeps [r * n_shard, (r+1) * n_shard) at arena offset `shard_off`.
// A gather job brings the flat range [lo, hi) into a local staging buffer (element lo lands at
// dst[0]). The range is cut into progress slots of `slot_elems` elements; a copy CTA owns every
// n_copy-th slot, moves it with TMA bulk copies (peer or local shard -> shared-memory ring -> local
// staging buffer, no multicast) and then raises the slot's epoch flag, which the GEMM producer of
// the same kernel (or nobody, for a stand-alone gather) acquires before its TMA loads touch the slot.
//
// The reference has no parameter sharding on the device; its plan only prices a per-layer
// ALL_GATHER in front of the first GEMM of a layer (src/model.c:442-451).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "../kernels/sm100.cuh"
#include "peer.cuh"
#include "signals.h"

namespace cai {

constexpr int kGatherRing = 6;                 // ring slots of kGatherPiece bytes
constexpr uint32_t kGatherPiece = 32768;       // bytes per bulk copy
constexpr int kGatherRingBytes = kGatherRing * static_cast<int>(kGatherPiece);

struct GatherJob {
    unsigned long long shard_off;  // arena offset of the parameter shard (same on every member)
    long long n_shard;             // elements per member
    long long lo, hi;              // flat element range to stage (multiples of 8)
    __nv_bfloat16* dst;            // local staging buffer
    long long slot_elems;          // elements per progress flag (multiple of 8)
    int nslots;                    // ceil((hi - lo) / slot_elems), at most kSigLocalSlots
    int reverse;                   // 1: stage the top of the range first (backward pass order)
    int n_copy;                    // CTAs that run the copy role
    int group_kind;                // signal region that holds the progress flags
};

// flag word of progress slot s
__device__ __forceinline__ uint32_t* gather_flag(const PeerTable& pt, const GatherJob& g, int s) {
    return sig_word(pt, pt.rank, g.group_kind, kSigLocal + s);
}

// Runs in ONE thread of copy CTA `cta` (0 <= cta < n_copy). ring: kGatherRingBytes of shared memory
// (16-byte aligned), bars: kGatherRing mbarriers. Returns false after a bounded wait ran out.
__device__ __forceinline__ bool gather_copy_role(const PeerTable& pt, const GatherJob& g, int cta, uint32_t epoch, uint8_t* ring,
                                                 uint64_t* bars, int* status) {
    volatile int no_abort = 0;
    for (int i = 0; i < kGatherRing; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
    uint32_t n_load = 0, n_store = 0;        // pieces loaded / stored so far (ring slot = n % kGatherRing)
    uint32_t bytes_of[kGatherRing];
    uint8_t* dst_of[kGatherRing];
    constexpr uint32_t kLag = kGatherRing - 2;  // loads in flight ahead of the store
    auto store_one = [&]() -> bool {
        const uint32_t slot = n_store % kGatherRing;
        if (!mbar_wait(&bars[slot], (n_store / kGatherRing) & 1, &no_abort, status, CAI_DEV_TIMEOUT_TMA_FULL)) return false;
        bulk_store(dst_of[slot], ring + slot * kGatherPiece, bytes_of[slot]);
        tma_store_commit();
        ++n_store;
        return true;
    };
    for (int k = cta; k < g.nslots; k += g.n_copy) {
        const int s = g.reverse ? g.nslots - 1 - k : k;
        long long a = g.lo + static_cast<long long>(s) * g.slot_elems;
        const long long b = a + g.slot_elems < g.hi ? a + g.slot_elems : g.hi;
        while (a < b) {
            // a piece never crosses a shard boundary and is at most kGatherPiece bytes
            const int owner = static_cast<int>(a / g.n_shard);
            const long long shard_end = (static_cast<long long>(owner) + 1) * g.n_shard;
            long long e = b < shard_end ? b : shard_end;
            if (e - a > static_cast<long long>(kGatherPiece / 2)) e = a + kGatherPiece / 2;
            const uint32_t bytes = static_cast<uint32_t>(e - a) * 2;
            const uint32_t slot = n_load % kGatherRing;
            if (n_load >= kGatherRing) bulk_wait_read1();  // the store that last used this ring slot has read it
            mbar_expect_tx(&bars[slot], bytes);
            bulk_load(ring + slot * kGatherPiece, pt.base[owner] + g.shard_off + (a - static_cast<long long>(owner) * g.n_shard) * 2, bytes,
                      &bars[slot]);
            bytes_of[slot] = bytes;
            dst_of[slot] = reinterpret_cast<uint8_t*>(g.dst + (a - g.lo));
            ++n_load;
            if (n_load - n_store > kLag && !store_one()) return false;
            a = e;
        }
        while (n_store < n_load)
            if (!store_one()) return false;
        tma_store_wait0();
        fence_proxy_async_all();
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(gather_flag(pt, g, s)), "r"(epoch) : "memory");
    }
    return true;
}

// Acquire-wait (bounded) until the progress slots covering staged elements [x, y) are there.
// Ends with the proxy fence a following TMA load needs. Returns false when the limit ran out.
__device__ __forceinline__ bool gather_wait_range(const PeerTable& pt, const GatherJob& g, long long x, long long y, uint32_t epoch,
                                                  int* status) {
    const int s0 = static_cast<int>(x / g.slot_elems);
    int s1 = static_cast<int>((y - 1) / g.slot_elems);
    if (s1 >= g.nslots) s1 = g.nslots - 1;
    for (int s = s0; s <= s1; ++s) {
        const uint32_t* flag = gather_flag(pt, g, s);
        bool seen = false, timed_out = false;
        // the copy CTA that raises this flag waits on a peer itself: give it its whole limit and a little more
        const uint64_t t0 = global_timer_ns(), limit = peer_wait_limit_ns(status) * 5 / 4;
        for (uint32_t it = 0; !seen; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            seen = static_cast<int32_t>(v - epoch) >= 0;
            if (!seen && !peer_spin_continue(it, t0, limit, status, &timed_out)) break;
        }
        if (!seen) {
            if (timed_out) atomicCAS(status, 0, CAI_DEV_TIMEOUT_PEER_FLAG);
            return false;
        }
    }
    fence_proxy_async_all();
    return true;
}

}  // namespace cai
