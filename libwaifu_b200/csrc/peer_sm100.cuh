// A barrier among the GPUs of one box, optionally carrying a maximum per row: the few microseconds
// between the kernels of a split linear that would otherwise be a library collective each.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerHeaderWords = 64;            // 256 bytes: word 0 is the flag, the payload follows
constexpr uint32_t kPeerDefaultPolls = 2000000; // about two seconds of polling before the wait gives up
constexpr uint32_t kStatusPeerTimeout = 0x61;   // a peer never signalled within the limit

// Every rank owns a mailbox, an int32 matrix (n_ranks, ld) with ld >= kPeerHeaderWords + rows, mapped
// into every peer; row j of it is written by rank j alone. One call, made by every rank with the
// same `epoch` (larger than at any call before on these mailboxes, which start zeroed):
//   1. if row_amax: writes its `rows` values (non-negative floats, as their bit patterns) into the
//      payload of row `rank` of every rank's mailbox;
//   2. orders everything this GPU wrote before (earlier kernels of the stream included) ahead of
//      a release store of `epoch` into word 0 of row `rank` of every rank's mailbox;
//   3. waits, acquiring, until word 0 of every row of its own mailbox has reached `epoch`; at most
//      max_polls polls per peer, after which it records kStatusPeerTimeout in *status and returns
//      with row_amax as it was;
//   4. if row_amax: row_amax[i] = the largest of the n_ranks payloads at i.
// One block; nothing in it waits on another launch of this GPU.
struct PeerExchangeArgs {
  int32_t *mailbox[kPeerMaxRanks];
  int n_ranks, rank;
  int64_t ld;
  int32_t epoch;
  float *row_amax;  // or nullptr: barrier only
  int rows;
  uint32_t max_polls;
  uint32_t *status;
  cudaStream_t stream;
};

cudaError_t peer_exchange(const PeerExchangeArgs &a);

}  // namespace flsm100
