// peer.cuh - what a fused compute+collective kernel knows about its communicator: the base
// address of every member's arena (mapped into this process over CUDA IPC, so an arena offset is
// valid on every rank) and the layout of the signal words inside each arena.
//
// Signal words are epoch counters that only grow: a waiter looks for "value >= epoch" with a
// wrap-safe signed difference, nothing is ever reset, so a late reader can never miss a signal
// and CUDA-graph replays need no host-side bookkeeping. The epoch of a launch is a per-step base
// read from device memory (refreshed by the host before every step) plus a sequence number that
// is fixed per op in the plan. All waits are bounded (sm100.cuh) and report through the status
// word instead of hanging.
#pragma once

#include <stdint.h>

#include "../kernels/sm100.cuh"
#include "signals.h"

namespace cai {

struct PeerTable {
    uint8_t* base[kMaxPeers];  // arena base of group member i as mapped in THIS process (base[rank] is local)
    int rank;
    int size;
    unsigned long long sig_off;  // byte offset of the signal block inside every arena
};

__device__ __forceinline__ uint32_t* sig_word(const PeerTable& pt, int member, int kind, uint32_t index) {
    return reinterpret_cast<uint32_t*>(pt.base[member] + pt.sig_off + static_cast<size_t>(kind) * kSigBytesPerKind) +
           static_cast<size_t>(index) * kSigWordStride;
}

// Publish `epoch` in slot `index` of every member (including this rank). Call from one thread,
// after the data the signal stands for has been written by this thread or made visible to it.
__device__ __forceinline__ void signal_all(const PeerTable& pt, int kind, uint32_t index, uint32_t epoch) {
    __threadfence_system();
    for (int m = 0; m < pt.size; ++m) st_release_sys(sig_word(pt, m, kind, index), epoch);
}

// Wait until every member has published `epoch` in its slot of region `first` of MY arena.
__device__ __forceinline__ bool wait_all(const PeerTable& pt, int kind, uint32_t first, uint32_t epoch, int* status) {
    for (int m = 0; m < pt.size; ++m)
        if (!wait_flag_ge(sig_word(pt, pt.rank, kind, first + m), epoch, status)) return false;
    return true;
}

}  // namespace cai
