// Layout of a rank's peer-exchange buffer for the fused tensor-parallel reduction (identical on
// every rank; the buffer is allocated by the tensor-parallel library and mapped into the peers
// through CUDA IPC).  Values travel as 8-byte {FP32 value, launch epoch} pairs: an aligned
// 8-byte store is a single transaction, so a pair is its own arrival flag.
#pragma once
#include <cstddef>

namespace nvfp4 {
namespace xchg {

constexpr int kMaxWorld = 8;
constexpr int kMaxTokens = 16;                 // tokens the fused reduction takes (the GEMV regime)
constexpr size_t kStatusOff = 0;               // sticky status word (0 = no wait ever ran out)
constexpr size_t kEpochOff = 64;               // launch counter, advanced by the kernels themselves (graph replays stay valid)
constexpr size_t kDoneOff = 128;               // CTAs finished in the current launch
constexpr size_t kSlotsOff = 4096;             // [2 sets][world][slot_pairs] pairs, written by the peers
constexpr long long kWaitClocks = 2000000000LL;   // about a second

inline size_t buffer_bytes(int world, int H) { return kSlotsOff + 2ull * world * kMaxTokens * H * 8; }

}  // namespace xchg
}  // namespace nvfp4
