// Host-side model of the peer-memory exchange protocol of ar_add_norm_kernel (two-shot form):
// C++ threads stand in for ranks, std::atomic words for the flags in peer-addressable
// staging, plain arrays for the staged data.  What the model checks is the PROTOCOL — the
// ordering of pushes, release/acquire flags, sequence numbers and the "done" guard on the
// reuse of the staging area — under adversarial scheduling, and what happens when a rank
// never arrives or arrives with a stale sequence number.  It mirrors the device code step by
// step (ar_norm.cu phases A-E) but shares no code with it.
//
//   protocol_model normal <ranks> <rows> <calls> <seed>   every rank must produce the exact sums
//   protocol_model absent <ranks> <rows>                  the last rank never calls
//   protocol_model stale  <ranks> <rows>                  rank 1 missed one call (its sequence lags)
// Exit code 0 when the expectations of the scenario hold; a line of JSON says what was seen.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int kMaxRanks = 8;
constexpr int kSliceWords = 8;        // words of a row that one rank reduces
constexpr uint32_t kPollLimit = 20000;
constexpr int kErrTimeout = -6;

struct RankMemory {                    // one rank's staging: flags + data, all written by peers
  std::atomic<uint32_t> done[kMaxRanks];
  std::vector<std::atomic<uint32_t>> pflag, sflag;  // [row][src]
  std::vector<uint32_t> scatter;       // [src][row][slice word]   partial slices pushed by peers
  std::vector<uint32_t> gather;        // [row][rank][slice word]  reduced slices pushed back
  uint32_t seq = 0;                    // local: collectives completed
  int status = 0;
  RankMemory(int R, int M) : pflag(M * kMaxRanks), sflag(M * kMaxRanks), scatter((size_t)R * M * kSliceWords),
                             gather((size_t)M * R * kSliceWords) {
    for (auto& d : done) d.store(0);
    for (auto& f : pflag) f.store(0);
    for (auto& f : sflag) f.store(0);
  }
};

uint32_t partial_word(uint32_t call, int rank, int row, int word) {
  return (call * 2654435761u) ^ (uint32_t)(rank * 97 + row * 31 + word * 7 + 1);
}

bool wait_ge(const std::atomic<uint32_t>& f, uint32_t target) {
  for (uint32_t it = 0; it < kPollLimit; ++it) {
    if ((int32_t)(f.load(std::memory_order_acquire) - target) >= 0) return true;
    if (it > 64) std::this_thread::yield();
  }
  return false;
}

struct World {
  int R, M;
  std::vector<RankMemory*> mem;
};

// One collective on rank `me`; `call` is the data generation this rank believes it is in.
// out[row][rank][word] receives the reduced rows.  Returns 0 or kErrTimeout.
int collective(World& w, int me, uint32_t call, std::vector<uint32_t>& out, std::mt19937& rng, bool jitter) {
  const int R = w.R, M = w.M;
  RankMemory& my = *w.mem[me];
  const uint32_t seq = my.seq, target = seq + 1;
  auto nap = [&] { if (jitter && rng() % 4 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 50)); };
  bool ok = true;
  for (int row = 0; row < M && ok; ++row) {   // the CTAs of a rank never wait for one another: any order is legal
    // A. peers are done reading the staging of the previous collective
    for (int q = 0; q < R && ok; ++q)
      if (q != me) ok = wait_ge(my.done[q], seq);
    if (!ok) break;
    nap();
    // B. push every other rank's slice of this row's partial into that rank's staging, then the flag
    for (int q = 0; q < R; ++q) {
      if (q == me) continue;
      for (int k = 0; k < kSliceWords; ++k)
        w.mem[q]->scatter[((size_t)me * M + row) * kSliceWords + k] = partial_word(call, me, row, q * kSliceWords + k);
      w.mem[q]->pflag[row * kMaxRanks + me].store(target, std::memory_order_release);
    }
    nap();
    // C. wait for the peers' slices, sum in rank order, push the reduced slice to everybody
    for (int q = 0; q < R && ok; ++q)
      if (q != me) ok = wait_ge(my.pflag[row * kMaxRanks + q], target);
    if (!ok) break;
    uint32_t red[kSliceWords];
    for (int k = 0; k < kSliceWords; ++k) {
      uint32_t acc = 0;
      for (int src = 0; src < R; ++src)
        acc += src == me ? partial_word(call, me, row, me * kSliceWords + k)
                         : my.scatter[((size_t)src * M + row) * kSliceWords + k];
      red[k] = acc;
      out[((size_t)row * R + me) * kSliceWords + k] = acc;
    }
    nap();
    for (int q = 0; q < R; ++q) {
      if (q == me) continue;
      for (int k = 0; k < kSliceWords; ++k) w.mem[q]->gather[((size_t)row * R + me) * kSliceWords + k] = red[k];
      w.mem[q]->sflag[row * kMaxRanks + me].store(target, std::memory_order_release);
    }
    // D. the slices reduced elsewhere
    for (int q = 0; q < R && ok; ++q)
      if (q != me) ok = wait_ge(my.sflag[row * kMaxRanks + q], target);
    if (!ok) break;
    for (int q = 0; q < R; ++q)
      if (q != me)
        for (int k = 0; k < kSliceWords; ++k)
          out[((size_t)row * R + q) * kSliceWords + k] = my.gather[((size_t)row * R + q) * kSliceWords + k];
  }
  if (!ok) my.status = kErrTimeout;
  // E. this rank is done with call `target` (published even after a timeout, as the kernel does)
  my.seq = target;
  for (int q = 0; q < R; ++q)
    if (q != me) w.mem[q]->done[me].store(target, std::memory_order_release);
  return ok ? 0 : kErrTimeout;
}

uint32_t expected(int R, uint32_t call, int row, int word) {
  uint32_t acc = 0;
  for (int r = 0; r < R; ++r) acc += partial_word(call, r, row, word);
  return acc;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const std::string mode = argv[1];
  const int R = atoi(argv[2]), M = atoi(argv[3]);
  const int calls = mode == "normal" && argc > 4 ? atoi(argv[4]) : 1;
  const unsigned seed = argc > 5 ? (unsigned)atoi(argv[5]) : 1u;
  if (R < 2 || R > kMaxRanks || M < 1) return 2;
  World w{R, M, {}};
  for (int r = 0; r < R; ++r) w.mem.push_back(new RankMemory(R, M));
  if (mode == "stale") {
    // everybody except rank 1 has completed one collective more than rank 1 knows of: their
    // counts and the "done" words they published say 1, rank 1's say 0
    for (int me = 0; me < R; ++me) {
      if (me == 1) continue;
      w.mem[me]->seq = 1;
      for (int q = 0; q < R; ++q)
        if (q != me) w.mem[q]->done[me].store(1);
    }
  }
  std::vector<int> wrong(R, 0), timeouts(R, 0);
  std::vector<std::thread> threads;
  const auto t0 = std::chrono::steady_clock::now();
  for (int me = 0; me < R; ++me) {
    threads.emplace_back([&, me] {
      std::mt19937 rng(seed * 1000 + me);
      std::vector<uint32_t> out((size_t)M * R * kSliceWords);
      if (mode == "absent" && me == R - 1) return;        // never arrives
      for (int c = 0; c < calls; ++c) {
        std::fill(out.begin(), out.end(), 0u);
        const uint32_t call = w.mem[me]->seq;                // the data generation = the rank's own count
        const int rc = collective(w, me, call, out, rng, mode == "normal");
        if (rc) { ++timeouts[me]; continue; }
        for (int row = 0; row < M; ++row)
          for (int k = 0; k < R * kSliceWords; ++k)
            if (out[(size_t)row * R * kSliceWords + k] != expected(R, call, row, k)) ++wrong[me];
      }
    });
  }
  for (auto& t : threads) t.join();
  const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  int n_wrong = 0, n_to = 0, ranks_to = 0;
  for (int r = 0; r < R; ++r) { n_wrong += wrong[r]; n_to += timeouts[r]; ranks_to += timeouts[r] > 0; }
  printf("{\"mode\": \"%s\", \"ranks\": %d, \"rows\": %d, \"calls\": %d, \"wrong_words\": %d, \"timeouts\": %d, "
         "\"ranks_timed_out\": %d, \"seconds\": %.3f}\n", mode.c_str(), R, M, calls, n_wrong, n_to, ranks_to, secs);
  bool pass = false;
  if (mode == "normal") pass = n_wrong == 0 && n_to == 0;
  // a missing rank: every rank that did call gives up (bounded) and says so; nobody hangs
  if (mode == "absent") pass = ranks_to == R - 1 && secs < 30.0;
  // a rank one call behind: its peers never see the flags they wait for and report it
  if (mode == "stale") pass = ranks_to >= R - 1 && secs < 30.0;
  for (auto* m : w.mem) delete m;
  return pass ? 0 : 1;
}
