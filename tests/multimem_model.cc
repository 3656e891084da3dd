// Host-side model of the switch-reduction exchange (mm_ar_add_norm_kernel, ar_multimem.cu): one
// C++ thread per (rank, batch row) stands in for a CTA, std::atomic words for the arrival
// counters of every rank's window, plain arrays for the partial and gather areas.  A
// "multicast" add or store is delivered to the ranks one after the other, in random order and
// with random pauses, as a switch may.  What the model checks is the PROTOCOL, under
// adversarial scheduling:
//   * targets derived from the counters as they stand before a CTA's own arrival (no
//     sequence number, nothing ever reset), with calls of DIFFERENT row counts in one run;
//   * the arrival signalled by the producing GEMM's last CTA instead (local call count x R);
//   * ONE partial area and ONE gather area per rank reused by consecutive calls: a rank
//     overwrites its partial as soon as its own kernel is complete;
//   * a rank that never arrives: every wait is bounded and reports.
// It mirrors the device code phase by phase (A arrival, B reduce + deliver, C gathered,
// D read the full row) but shares no code with it.
//
//   multimem_model normal  <ranks> <max rows> <calls> <seed> <gemm_signals 0|1>
//   multimem_model absent  <ranks> <rows>
// Exit code 0 when the expectations of the scenario hold; a line of JSON says what was seen.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include <pthread.h>

namespace {

constexpr int kMaxRanks = 8, kMaxRows = 16;
constexpr int kSliceWords = 4;          // words of a row that one rank reduces
constexpr uint32_t kPollLimit = 200000;

struct Window {                         // one rank's window
  std::atomic<uint32_t> ready[kMaxRows], gathered[kMaxRows], ready_all;
  uint32_t gemm_calls = 0;              // local only
  std::vector<uint32_t> partial, gather;  // [row][R * kSliceWords]
  Window(int R) : partial(kMaxRows * R * kSliceWords), gather(kMaxRows * R * kSliceWords) {
    for (auto& c : ready) c.store(0);
    for (auto& c : gathered) c.store(0);
    ready_all.store(0);
  }
};

struct World {
  int R;
  std::vector<Window*> win;
};

uint32_t partial_word(uint32_t call, int rank, int row, int word) {
  return (call * 2654435761u) ^ (uint32_t)(rank * 97 + row * 31 + word * 7 + 1);
}

void nap(std::mt19937& rng, bool jitter) {
  if (jitter && rng() % 3 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 40));
}

// a multicast operation reaches the ranks one by one, in any order
template <typename F>
void to_all_ranks(World& w, std::mt19937& rng, bool jitter, F f) {
  std::vector<int> order(w.R);
  std::iota(order.begin(), order.end(), 0);
  std::shuffle(order.begin(), order.end(), rng);
  for (int q : order) {
    nap(rng, jitter);
    f(*w.win[q]);
  }
}

bool wait_ge(const std::atomic<uint32_t>& c, uint32_t target) {
  for (uint32_t it = 0; it < kPollLimit; ++it) {
    if ((int32_t)(c.load(std::memory_order_acquire) - target) >= 0) return true;
    if (it > 64) std::this_thread::yield();
  }
  return false;
}

// the kernel of one CTA: rank `me`, batch row `row`.  0 = ok, 1 = a wait ran out, 2 = wrong sums
int cta(World& w, int me, int row, uint32_t call, bool gemm_signals, std::mt19937& rng, bool jitter) {
  const int R = w.R;
  Window& my = *w.win[me];
  const uint32_t mask = ~(uint32_t)(R - 1);
  // targets from the counters as they stand BEFORE this CTA's own arrival
  const uint32_t target_c = (my.gathered[row].load(std::memory_order_acquire) & mask) + (uint32_t)R;
  bool ok;
  if (gemm_signals) {
    ok = wait_ge(my.ready_all, my.gemm_calls * (uint32_t)R);
  } else {
    const uint32_t target_a = (my.ready[row].load(std::memory_order_acquire) & mask) + (uint32_t)R;
    to_all_ranks(w, rng, jitter, [&](Window& q) { q.ready[row].fetch_add(1, std::memory_order_release); });
    ok = wait_ge(my.ready[row], target_a);
  }
  if (!ok) return 1;
  nap(rng, jitter);
  // B. this rank's slice: the sum over all ranks' partials, delivered to every rank's gather area
  uint32_t red[kSliceWords];
  for (int k = 0; k < kSliceWords; ++k) {
    uint32_t acc = 0;
    for (int q = 0; q < R; ++q) acc += w.win[q]->partial[(row * R + me) * kSliceWords + k];
    red[k] = acc;
  }
  to_all_ranks(w, rng, jitter, [&](Window& q) {
    for (int k = 0; k < kSliceWords; ++k) q.gather[(row * R + me) * kSliceWords + k] = red[k];
  });
  // C. release, then the arrival on `gathered`
  std::atomic_thread_fence(std::memory_order_release);
  to_all_ranks(w, rng, jitter, [&](Window& q) { q.gathered[row].fetch_add(1, std::memory_order_release); });
  if (!wait_ge(my.gathered[row], target_c)) return 1;
  // D. the full row
  for (int s = 0; s < R; ++s)
    for (int k = 0; k < kSliceWords; ++k) {
      uint32_t want = 0;
      for (int q = 0; q < R; ++q) want += partial_word(call, q, row, s * kSliceWords + k);
      if (my.gather[(row * R + s) * kSliceWords + k] != want) return 2;
    }
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const std::string mode = argv[1];
  const int R = atoi(argv[2]), max_rows = atoi(argv[3]);
  const int calls = mode == "normal" && argc > 4 ? atoi(argv[4]) : 1;
  const unsigned seed = argc > 5 ? (unsigned)atoi(argv[5]) : 1u;
  const bool gemm_signals = argc > 6 && atoi(argv[6]) != 0;
  if (R < 2 || R > kMaxRanks || (R & (R - 1)) || max_rows < 1 || max_rows > kMaxRows) return 2;
  World w{R, {}};
  for (int r = 0; r < R; ++r) w.win.push_back(new Window(R));
  // rows of every call: the same sequence on all ranks, varying from call to call
  std::vector<int> rows_of(calls);
  {
    std::mt19937 g(seed);
    for (int c = 0; c < calls; ++c) rows_of[c] = mode == "normal" ? 1 + (int)(g() % max_rows) : max_rows;
  }
  const bool absent = mode == "absent";
  std::vector<pthread_barrier_t> rank_bar(R);
  for (auto& b : rank_bar) pthread_barrier_init(&b, nullptr, max_rows);
  std::atomic<int> wrong{0}, timeouts{0};
  std::vector<std::atomic<int>> rank_timed_out(R);
  for (auto& t : rank_timed_out) t.store(0);
  std::vector<std::thread> threads;
  const auto t0 = std::chrono::steady_clock::now();
  for (int me = 0; me < R; ++me) {
    if (absent && me == R - 1) continue;            // never launches anything
    for (int row = 0; row < max_rows; ++row) {
      threads.emplace_back([&, me, row] {
        std::mt19937 rng(seed * 7919 + me * 131 + row);
        Window& my = *w.win[me];
        for (int c = 0; c < calls; ++c) {
          const int M = rows_of[c];
          if (row == 0) {
            // the producing GEMM of this rank: overwrites the partial area (the previous call's
            // kernel has completed on THIS rank; peers may be anywhere), then signals if asked
            for (int r2 = 0; r2 < M; ++r2)
              for (int k = 0; k < R * kSliceWords; ++k) my.partial[r2 * R * kSliceWords + k] = partial_word(c, me, r2, k);
            if (gemm_signals) {
              my.gemm_calls += 1;
              std::atomic_thread_fence(std::memory_order_release);
              to_all_ranks(w, rng, !absent, [&](Window& q) { q.ready_all.fetch_add(1, std::memory_order_release); });
            }
          }
          pthread_barrier_wait(&rank_bar[me]);     // kernel boundary: the exchange kernel starts
          if (row < M) {
            const int rc = cta(w, me, row, (uint32_t)c, gemm_signals, rng, !absent);
            if (rc == 1) { ++timeouts; rank_timed_out[me].store(1); }
            if (rc == 2) ++wrong;
          }
          pthread_barrier_wait(&rank_bar[me]);     // kernel complete on this rank
        }
      });
    }
  }
  for (auto& t : threads) t.join();
  const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  int ranks_to = 0;
  for (auto& t : rank_timed_out) ranks_to += t.load();
  printf("{\"mode\": \"%s\", \"ranks\": %d, \"max_rows\": %d, \"calls\": %d, \"gemm_signals\": %d, \"wrong_rows\": %d, "
         "\"timeouts\": %d, \"ranks_timed_out\": %d, \"seconds\": %.3f}\n",
         mode.c_str(), R, max_rows, calls, gemm_signals ? 1 : 0, wrong.load(), timeouts.load(), ranks_to, secs);
  bool pass = false;
  if (mode == "normal") pass = wrong.load() == 0 && timeouts.load() == 0;
  if (mode == "absent") pass = ranks_to == R - 1 && wrong.load() == 0 && secs < 60.0;
  for (auto* p : w.win) delete p;
  return pass ? 0 : 1;
}
