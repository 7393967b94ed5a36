// Host-side simulation of the state-exchange protocol (relay_kernels.cu) using
// the kernel's own index arithmetic (lasp_b200/csrc/exchange_layout.h).
//
// All ranks' buffers live in this process.  Each step runs every rank's push
// CTAs, then every rank's gather CTAs, thread by thread, exactly as the kernel
// partitions them, and checks that
//   * every destination word whose decay power is above the cut-off is written exactly once per step
//     with the step number, and no other word is written or read,
//   * every gathered element equals sum_q a^(me-1-q) total_q (same Horner order),
//   * acknowledgements land in the words the pushers later wait on, and the wait
//     of step s (>= 3) finds the value s-2 already there.
// usage: exchange_sim <ranks> <elems> <steps>   -> exit 0 and "ok", or a message
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "exchange_layout.h"

using namespace lasp::xl;

struct Word { float value; uint32_t step; };

struct Rank {
  std::vector<Word> slots;       // [2][ranks][elems]
  std::vector<uint32_t> acks;    // [ranks * kSlices * kAckStride]
  std::vector<float> total, x_in;
  std::vector<int> writes;       // per slot word: writes in the current step
  uint32_t counter = 0;
};

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const int ranks = atoi(argv[1]);
  const long long elems = atoll(argv[2]);
  const int steps = atoi(argv[3]);
  const int h = 3;
  const long long de = elems / 6 > 0 && (elems % 6 == 0) ? elems / 6 : elems;  // pretend b*h = 6 when it divides
  const float s[3] = {0.0f, 0.001f, 0.15f};   // the last head reaches the next rank only (s n = 15 per hop... 2 hops = 30 > cut-off)
  const int n = 100;
  std::vector<Rank> R(ranks);
  for (auto& r : R) {
    r.slots.assign(2 * ranks * elems, Word{0.f, 0u});
    r.acks.assign(ranks * kSlices * kAckStride, 0u);
    r.total.resize(elems);
    r.x_in.assign(elems, 0.f);
    r.writes.assign(2 * ranks * elems, 0);
  }
  for (int step_i = 1; step_i <= steps; ++step_i) {
    for (int me = 0; me < ranks; ++me)
      for (long long i = 0; i < elems; ++i) R[me].total[i] = (float)((me + 1) * 1000 + step_i) + 0.001f * (float)(i % 977);
    for (auto& r : R) std::fill(r.writes.begin(), r.writes.end(), 0);
    // ---- push phase
    for (int me = 0; me < ranks; ++me) {
      const uint32_t step = R[me].counter + 1;
      if ((int)step != step_i) { printf("rank %d: step %u != %d\n", me, step, step_i); return 1; }
      const int parity = step & 1, n_dst = ranks - 1 - me, parts = push_parts(n_dst);
      for (int block = 0; block < push_ctas(n_dst); ++block) {
        int di, slice, part;
        push_decode(block, parts, &di, &slice, &part);
        const int dst = me + 1 + di;
        if (dst >= ranks || slice >= kSlices) { printf("bad decode\n"); return 1; }
        if (needs_ack_wait(step) && R[me].acks[ack_index(dst, slice)] < step - 2) {
          printf("rank %d step %u: ack of (dst %d, slice %d) is %u, pusher would wait\n", me, step, dst, slice,
                 R[me].acks[ack_index(dst, slice)]);
          return 1;
        }
        long long lo, hi;
        part_bounds(elems, slice, parts, part, &lo, &hi);
        const long long off = slot_offset(parity, ranks, me, elems);
        for (int t = 0; t < kThreads; ++t)
          for (long long base = lo + (long long)t * kVec; base < hi; base += kThreads * kVec * 4)
            for (int u = 0; u < 4; ++u) {
              const long long el = base + (long long)u * kThreads * kVec;
              if (el >= hi) continue;
              if (!reaches(s[(el / de) % h] * (float)n, di)) continue;   // one head per group of kVec elements
              for (int j = 0; j < kVec; ++j) {
                if (el + j >= elems) { printf("push out of range\n"); return 1; }
                R[dst].slots[off + el + j] = Word{R[me].total[el + j], step};
                R[dst].writes[off + el + j]++;
              }
            }
      }
    }
    // every word a gatherer will read was written exactly once
    for (int me = 1; me < ranks; ++me)
      for (int q = 0; q < me; ++q)
        for (long long i = 0; i < elems; ++i)
          if (R[me].writes[slot_offset(step_i & 1, ranks, q, elems) + i] !=
              (reaches(s[(i / de) % h] * (float)n, me - 1 - q) ? 1 : 0)) {
            printf("rank %d: word of source %d element %lld written %d times\n", me, q, i,
                   R[me].writes[slot_offset(step_i & 1, ranks, q, elems) + i]);
            return 1;
          }
    // ---- gather phase
    for (int me = 0; me < ranks; ++me) {
      const uint32_t step = R[me].counter + 1;
      const int parity = step & 1, n_src = me;
      std::vector<int> seen(elems, 0);
      for (int gi = 0; gi < gather_ctas(n_src); ++gi) {
        int slice, part;
        gather_decode(gi, &slice, &part);
        long long lo, hi;
        part_bounds(elems, slice, kGatherCtas, part, &lo, &hi);
        const long long off = slot_offset(parity, ranks, 0, elems);
        for (int t = 0; t < kThreads; ++t)
          for (long long el = lo + (long long)t * kVec; el < hi; el += kThreads * kVec)
            for (int j = 0; j < kVec; ++j) {
              const float a = expf(-s[((el + j) / de) % h] * (float)n);
              float acc = 0.f;
              for (int q = 0; q < n_src; ++q) {
                if (!reaches(s[((el + j) / de) % h] * (float)n, me - 1 - q)) { acc *= a; continue; }
                const Word w = R[me].slots[off + (long long)q * elems + el + j];
                if (w.step != step) { printf("rank %d: stale word (step %u, want %u)\n", me, w.step, step); return 1; }
                acc = fmaf(a, acc, w.value);
              }
              R[me].x_in[el + j] = acc;
              seen[el + j]++;
            }
        if (part == kGatherCtas - 1)  // last part of the slice: acknowledge to every source
          for (int q = 0; q < n_src; ++q) R[q].acks[ack_index(me, slice)] = step;
      }
      if (n_src > 0)
        for (long long i = 0; i < elems; ++i) {
          if (seen[i] != 1) { printf("rank %d: element %lld gathered %d times\n", me, i, seen[i]); return 1; }
          const float a = expf(-s[(i / de) % h] * (float)n);
          double ref = 0;
          for (int q = 0; q < n_src; ++q) ref = ref * a + R[q].total[i];
          if (fabs(ref - R[me].x_in[i]) > 1e-3 * fabs(ref) + 1e-3) { printf("rank %d: wrong sum at %lld\n", me, i); return 1; }
        }
      R[me].counter = step;
    }
  }
  printf("ok\n");
  return 0;
}
