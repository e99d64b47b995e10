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

#ifdef __CUDACC__
__device__ __forceinline__ uint4 ld_words(const uint2* p) {  // two staging words
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Reads the two words again until both carry `tag` (bounded: two seconds).
__device__ __forceinline__ void settle(uint4& v, const uint2* p, uint32_t tag, int* status) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; v.y != tag || v.w != tag; ++i) {
    v = ld_words(p);
    if ((i & 63u) == 63u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) {
        atomicOr(status, 1);
        v = make_uint4(0u, tag, 0u, tag);
      }
    }
  }
}

// The partial sums of push `c` for 8 consecutive elements starting at element `i` of a slot,
// added over the ranks in rank order in fp32 and rounded to bf16 pairs.  `words` points at
// slot 0 of the half of push c; every rank's words are requested before any is checked.
__device__ __forceinline__ uint4 reduce_ranks(const uint2* words, long long slot, int tp, long long i, uint32_t c,
                                              int* status) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  uint4 v[2 * kTpMaxRanks];
#pragma unroll
  for (int j = 0; j < kTpMaxRanks; ++j) {
    if (j < tp) {
      const uint2* w = words + ((size_t)j * slot + i) / 2;
      v[2 * j] = ld_words(w);
      v[2 * j + 1] = ld_words(w + 2);
    }
  }
  auto lo16 = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto hi16 = [](uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); };
#pragma unroll
  for (int j = 0; j < kTpMaxRanks; ++j) {
    if (j < tp) {
      const uint2* w = words + ((size_t)j * slot + i) / 2;
      settle(v[2 * j], w, c + 1u, status);
      settle(v[2 * j + 1], w + 2, c + 1u, status);
      const uint4 lo = v[2 * j], hi = v[2 * j + 1];
      acc[0] += lo16(lo.x); acc[1] += hi16(lo.x);
      acc[2] += lo16(lo.z); acc[3] += hi16(lo.z);
      acc[4] += lo16(hi.x); acc[5] += hi16(hi.x);
      acc[6] += lo16(hi.z); acc[7] += hi16(hi.z);
    }
  }
  auto pack = [](float a, float b) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
    return d;
  };
  return make_uint4(pack(acc[0], acc[1]), pack(acc[2], acc[3]), pack(acc[4], acc[5]), pack(acc[6], acc[7]));
}
#endif

}  // namespace fdk
