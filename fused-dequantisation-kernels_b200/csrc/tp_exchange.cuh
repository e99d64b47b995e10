// Layout of a tensor-parallel exchange buffer (one per rank, mapped by all ranks):
//   [128, 132)   reduces completed by this rank so far = number c of the next push
//   [132, 136)   CTAs of the running reduce that have finished
//   [136, 140)   status: 1 = a reduce gave up waiting for a word
//   [256, ...)   staging, 8-byte words {two 16-bit partial sums, tag} [2 halves][tp][slot_elems / 2]:
//                push c of rank j writes slot j of half c & 1 on every rank with tag c + 1;
//                a word is valid for reduce c once its tag is c + 1
// Only [128, 256) is written locally and only [256, ...) remotely.
#pragma once
#include <cstddef>
#include <cstdint>

namespace fdk {

constexpr int kTpMaxRanks = 8;
constexpr size_t kTpSeqOffset = 128;
constexpr size_t kTpDoneOffset = 132;
constexpr size_t kTpStatusOffset = 136;
constexpr size_t kTpStageOffset = 256;

inline size_t tp_exchange_bytes(int tp, long long slot_elems) {
  return kTpStageOffset + (size_t)2 * tp * (size_t)slot_elems * 4;
}

}  // namespace fdk
