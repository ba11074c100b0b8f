// signals.h - layout of the signal block every arena carries for the fused compute+collective
// kernels (plain constants, shared by the plan compiler and the device code).
//
// Words are uint32 epoch counters, one per 32-byte sector. Each communicator kind owns a region:
//   entry[member]        "my input of this op is ready", written by a member into every peer
//   exit[member]         "I am done with your memory"
//   local[slot]          progress flags between CTAs of one GPU (all-gather staging)
//   tile[member][slot]   per-tile arrival flags of the GEMM -> reduce-scatter kernel
#pragma once

#include <stdint.h>

namespace cai {

constexpr int kMaxPeers = 8;
constexpr uint32_t kSigWordStride = 8;  // uint32 per flag (32 bytes)
constexpr uint32_t kSigEntry = 0;
constexpr uint32_t kSigExit = kSigEntry + kMaxPeers;
constexpr uint32_t kSigLocal = kSigExit + kMaxPeers;
constexpr uint32_t kSigLocalSlots = 1024;
constexpr uint32_t kSigTile = kSigLocal + kSigLocalSlots;
constexpr uint32_t kSigTileSlots = 1024;
constexpr uint32_t kSigWordsPerKind = kSigTile + kMaxPeers * kSigTileSlots;
constexpr uint32_t kSigBytesPerKind = kSigWordsPerKind * kSigWordStride * 4;
constexpr uint32_t kSigKinds = 4;  // TP, DP, PP, EP
constexpr uint32_t kSigBytes = kSigBytesPerKind * kSigKinds;

}  // namespace cai
