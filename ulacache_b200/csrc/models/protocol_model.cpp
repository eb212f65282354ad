// Host model of the peer-memory protocols, one thread per rank, for ThreadSanitizer.
//
// The kernels synchronise ranks with three idioms.  Each is restated here with std::atomic and the SAME memory
// orders, payloads as plain (non-atomic) memory, so that ThreadSanitizer checks what the orders are meant to give:
// no rank reads a payload before it is complete, and no rank overwrites a buffer another rank may still read.
//
//   1. flag barrier around a double-buffered payload exchange (peer_put + step_barrier_kernel, ipc.cu): payload
//      stores, a system fence, a release store of the step count into every peer's flag page; acquire polls of
//      this rank's page; the receive buffer of step s is reused at step s + 2.
//   2. reader-lifetime phases (lifetime_publish_kernel / lifetime_wait_kernel, collective.cu): an owner may
//      overwrite its pool only after every reader published ReadersRetired for the previous step; readers may read
//      only after ResidencyReady of this step.
//   3. tagged words (tagged_all_gather_kernel): 4 payload bytes and the 4-byte call index travel in ONE 8-byte
//      relaxed store; the receiver polls the word until the tag matches; slots rotate, no barrier.  Checked by
//      value (everything is atomic, so a wrong slot count shows as a wrong value or a wait that runs out).
//
// What is NOT modelled: the 128-byte line protocol relies on NVLink delivering an aligned 128-byte store whole,
// a property of the link that C++ atomics cannot express.
//
// Usage: protocol_model <scenario> [ranks] [steps]; scenarios: barrier, lifetime, tagged, and two
// deliberately broken ones: tagged-one-slot (must end with "timeout", exit code 3) and barrier-relaxed (must be
// reported by ThreadSanitizer).  Exit 0 = passed.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <thread>
#include <vector>

namespace {

constexpr int kMaxRanks = 8;
constexpr long kSpinLimit = 20000000;      // polls before a wait gives up (the kernels' cycle limit)

std::atomic<int> g_errors{0};
std::atomic<int> g_timeouts{0};

void jitter(std::mt19937& rng, int max_us) {
  const int us = static_cast<int>(rng() % (max_us + 1));
  if (us > 0) std::this_thread::sleep_for(std::chrono::microseconds(us));
}

bool wait_ge(const std::atomic<int32_t>& flag, int32_t want) {
  for (long i = 0; i < kSpinLimit; ++i) {
    if (flag.load(std::memory_order_acquire) >= want) return true;      // ld.acquire.sys
    if ((i & 63) == 63) std::this_thread::yield();
  }
  g_timeouts.fetch_add(1);
  return false;
}

// ---------------------------------------------------------------------------------- 1. barrier --
struct BarrierWorld {
  int ranks, words;
  std::vector<int32_t> recv;                                  // [rank][parity][src][words], plain memory
  std::unique_ptr<std::atomic<int32_t>[]> flags;              // [rank][src]
  int32_t* buf(int rank, int parity, int src) { return recv.data() + ((static_cast<size_t>(rank) * 2 + parity) * ranks + src) * words; }
};

void barrier_rank(BarrierWorld* w, int me, int steps, std::memory_order flag_order) {
  std::mt19937 rng(1234 + me);
  for (int s = 1; s <= steps; ++s) {
    const int parity = s & 1;
    for (int p = 0; p < w->ranks; ++p) {                       // peer_put: my block into every rank's buffer
      int32_t* dst = w->buf(p, parity, me);
      for (int i = 0; i < w->words; ++i) dst[i] = s * 1000 + me * 10 + (i & 7);
    }
    jitter(rng, 20);
    // (the kernel also issues __threadfence_system() first; ThreadSanitizer does not model stand-alone fences,
    // and the release store alone already orders the payload for it)
    for (int p = 0; p < w->ranks; ++p) w->flags[p * kMaxRanks + me].store(s, flag_order);            // st.release.sys
    for (int r = 0; r < w->ranks; ++r)
      if (!wait_ge(w->flags[me * kMaxRanks + r], s)) return;
    for (int r = 0; r < w->ranks; ++r) {                       // the consumer kernel reads what arrived
      const int32_t* src = w->buf(me, parity, r);
      for (int i = 0; i < w->words; ++i)
        if (src[i] != s * 1000 + r * 10 + (i & 7)) { g_errors.fetch_add(1); return; }
    }
    jitter(rng, me == 0 ? 60 : 5);                             // one slow rank
  }
}

// --------------------------------------------------------------------------------- 2. lifetime --
enum Phase { kSelectionsReady = 0, kResidencyReady = 1, kReadersRetired = 2 };

struct LifetimeWorld {
  int ranks, slots;
  std::vector<int32_t> pool;                                  // [owner][slots], plain
  std::vector<int32_t> selection;                             // [owner][reader]: slot the reader asks for, plain
  std::unique_ptr<std::atomic<int32_t>[]> page;               // [rank][phase][src]
  std::atomic<int32_t>& flag(int rank, int phase, int src) { return page[(rank * 3 + phase) * kMaxRanks + src]; }
};

void lifetime_publish(LifetimeWorld* w, int me, int phase, int epoch) {
  for (int r = 0; r < w->ranks; ++r) w->flag(r, phase, me).store(epoch, std::memory_order_release);
}

bool lifetime_wait(LifetimeWorld* w, int me, int phase, int epoch) {
  for (int r = 0; r < w->ranks; ++r)
    if (!wait_ge(w->flag(me, phase, r), epoch)) return false;
  return true;
}

void lifetime_rank(LifetimeWorld* w, int me, int steps) {
  std::mt19937 rng(99 + me);
  for (int s = 1; s <= steps; ++s) {
    // every reader tells every owner which slot it will read
    for (int o = 0; o < w->ranks; ++o) w->selection[(o * w->ranks + me)] = (s * 7 + me * 3 + o) % w->slots;
    lifetime_publish(w, me, kSelectionsReady, s);
    if (!lifetime_wait(w, me, kSelectionsReady, s)) return;
    // owner: readers of the previous step have retired (waited for at the end of that step), so the slots
    // may be overwritten: "promote" what was asked for
    for (int r = 0; r < w->ranks; ++r) {
      const int slot = w->selection[me * w->ranks + r];
      w->pool[me * w->slots + slot] = s * 100 + me;
    }
    jitter(rng, 15);
    lifetime_publish(w, me, kResidencyReady, s);
    if (!lifetime_wait(w, me, kResidencyReady, s)) return;
    // reader: read the slot it asked for from every owner's pool
    for (int o = 0; o < w->ranks; ++o) {
      const int slot = (s * 7 + me * 3 + o) % w->slots;
      if (w->pool[o * w->slots + slot] != s * 100 + o) { g_errors.fetch_add(1); return; }
    }
    jitter(rng, me == 1 ? 40 : 3);
    lifetime_publish(w, me, kReadersRetired, s);
    if (!lifetime_wait(w, me, kReadersRetired, s)) return;
  }
}

// ----------------------------------------------------------------------------------- 3. tagged --
struct TaggedWorld {
  int ranks, n, slots;
  std::unique_ptr<std::atomic<uint64_t>[]> slab;              // [rank][slot][src][n]
  std::atomic<uint64_t>& word(int rank, int slot, int src, int i) {
    return slab[((static_cast<size_t>(rank) * slots + slot) * ranks + src) * n + i];
  }
};

void tagged_rank(TaggedWorld* w, int me, int calls, bool slow_reader) {
  std::mt19937 rng(7 + me);
  for (uint32_t idx = 1; idx <= static_cast<uint32_t>(calls); ++idx) {
    const int slot = static_cast<int>((idx - 1) % w->slots);
    for (int i = 0; i < w->n; ++i) {
      const uint64_t v = (static_cast<uint64_t>(idx) << 32) | static_cast<uint32_t>(idx * 100000 + me * 1000 + i);
      for (int p = 0; p < w->ranks; ++p) w->word(p, slot, me, i).store(v, std::memory_order_relaxed);   // st.relaxed.sys.v2
    }
    if (slow_reader && me == 0) {
      // the slow reader of the broken configuration: it looks at its slab only after the peer has lapped it (the
      // peer's NEXT call has landed in the only slot), so the outcome does not depend on scheduling
      for (long spin = 0; spin < kSpinLimit; ++spin) {
        if (static_cast<uint32_t>(w->word(me, slot, 1, 0).load(std::memory_order_relaxed) >> 32) == idx + 1) break;
        if ((spin & 63) == 63) std::this_thread::yield();
      }
    } else {
      jitter(rng, 10);
    }
    for (int r = 0; r < w->ranks; ++r)
      for (int i = 0; i < w->n; ++i) {
        bool ok = false;
        uint64_t v = 0;
        for (long spin = 0; spin < kSpinLimit / 20; ++spin) {
          v = w->word(me, slot, r, i).load(std::memory_order_relaxed);
          if (static_cast<uint32_t>(v >> 32) == idx) { ok = true; break; }
          if ((spin & 63) == 63) std::this_thread::yield();
        }
        if (!ok) { g_timeouts.fetch_add(1); return; }
        if (static_cast<uint32_t>(v) != idx * 100000 + static_cast<uint32_t>(r) * 1000 + static_cast<uint32_t>(i)) {
          g_errors.fetch_add(1);
          return;
        }
      }
  }
}

template <class F>
void run_ranks(int ranks, F f) {
  std::vector<std::thread> t;
  for (int r = 0; r < ranks; ++r) t.emplace_back(f, r);
  for (auto& x : t) x.join();
}

}  // namespace

int main(int argc, char** argv) {
  const char* what = argc > 1 ? argv[1] : "barrier";
  const int ranks = argc > 2 ? std::atoi(argv[2]) : 4;
  const int steps = argc > 3 ? std::atoi(argv[3]) : 200;
  if (ranks < 2 || ranks > kMaxRanks || steps < 1) { std::fprintf(stderr, "ranks 2..8, steps >= 1\n"); return 2; }
  if (!std::strcmp(what, "barrier") || !std::strcmp(what, "barrier-relaxed")) {
    // "barrier-relaxed" publishes the flags with relaxed stores: a deliberately broken order that ThreadSanitizer
    // must report as a race on the payload (it shows the check is sensitive to the order under test)
    const std::memory_order order = std::strcmp(what, "barrier") ? std::memory_order_relaxed : std::memory_order_release;
    BarrierWorld w;
    w.ranks = ranks; w.words = 64;
    w.recv.assign(static_cast<size_t>(ranks) * 2 * ranks * w.words, 0);
    w.flags.reset(new std::atomic<int32_t>[ranks * kMaxRanks]);
    for (int i = 0; i < ranks * kMaxRanks; ++i) w.flags[i].store(0);
    run_ranks(ranks, [&](int r) { barrier_rank(&w, r, steps, order); });
  } else if (!std::strcmp(what, "lifetime")) {
    LifetimeWorld w;
    w.ranks = ranks; w.slots = 16;
    w.pool.assign(static_cast<size_t>(ranks) * w.slots, 0);
    w.selection.assign(static_cast<size_t>(ranks) * ranks, 0);
    w.page.reset(new std::atomic<int32_t>[ranks * 3 * kMaxRanks]);
    for (int i = 0; i < ranks * 3 * kMaxRanks; ++i) w.page[i].store(0);
    run_ranks(ranks, [&](int r) { lifetime_rank(&w, r, steps); });
  } else if (!std::strcmp(what, "tagged") || !std::strcmp(what, "tagged-one-slot")) {
    const bool broken = !std::strcmp(what, "tagged-one-slot");
    TaggedWorld w;
    w.ranks = broken ? 2 : ranks; w.n = 32; w.slots = broken ? 1 : 4;
    const size_t total = static_cast<size_t>(w.ranks) * w.slots * w.ranks * w.n;
    w.slab.reset(new std::atomic<uint64_t>[total]);
    for (size_t i = 0; i < total; ++i) w.slab[i].store(0);
    run_ranks(w.ranks, [&](int r) { tagged_rank(&w, r, broken ? 4 : steps, broken); });
  } else {
    std::fprintf(stderr, "unknown scenario %s\n", what);
    return 2;
  }
  const int e = g_errors.load(), t = g_timeouts.load();
  std::printf("%s: ranks=%d steps=%d errors=%d %s\n", what, ranks, steps, e, t ? "timeout" : "ok");
  if (e) return 1;
  return t ? 3 : 0;
}
