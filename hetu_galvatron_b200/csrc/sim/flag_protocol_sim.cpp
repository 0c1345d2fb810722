// Host-side simulator of the peer-memory signalling protocol of include/gv_comm.cuh: ranks are threads, symmetric
// workspaces are host arrays, system-scope release stores / acquire loads are std::atomic release / acquire, and the
// payload is plain (non-atomic) memory so that a thread sanitizer build reports every access the protocol fails to
// order. It runs the two patterns the kernels use,
//
//   pull : every rank publishes a block for epoch e, announces e to all ranks, waits for every peer's announcement and
//          reads the peers' blocks (all-gather pull, KV gather, ZeRO-3 gather, A-operand gather of the fused GEMM);
//   push : every rank writes its contribution into slot[rank] of every OWNER's workspace, announces e, and each owner
//          waits for all announcements and sums its slots (GEMM -> reduce-scatter epilogue + slot reduction);
//
// with payload regions double buffered by epoch parity: a rank reuses the region of epoch e-2 at epoch e, which is safe
// because in epoch e-1 it waited for every peer's e-1 announcement, and a peer announces e-1 only after it finished
// with epoch e-2. `--single-buffer` removes the double buffering (one region for all epochs): readers then observe
// blocks of a later epoch, which the checker counts (this mode exists to show that the checker can see the hazard).
// Every wait is bounded, as on the device: `--drop-rank r --drop-epoch e` makes rank r stop at epoch e without
// announcing; the others' waits give up after the budget, record {site, src, epoch} and all threads still finish.
//
// The reference has no such tool (it has no in-kernel signalling at all).
//
//   g++ -std=c++17 -O1 -g -pthread [-fsanitize=thread] flag_protocol_sim.cpp -o flag_protocol_sim
//   ./flag_protocol_sim --ranks 4 --epochs 200 --mode pull|push [--seed S] [--single-buffer] [--drop-rank r --drop-epoch e]
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int kMaxRanks = 8;       // GV_MAX_RANKS
constexpr int kSlots = 16;         // GV_FLAG_SLOTS
constexpr int kBlock = 256;        // payload words per rank and epoch
constexpr int kSlotData = 3;       // flag slot used by the data exchange

struct Workspace {
  std::atomic<uint32_t> flags[kSlots * kMaxRanks];
  std::vector<uint32_t> payload;   // pull: [2][kBlock]; push: [2][world][kBlock]
};

struct ErrorWord {
  std::atomic<uint32_t> code{0};
  uint32_t site = 0, src = 0, epoch = 0;
};

struct Config {
  int ranks = 4, epochs = 100, drop_rank = -1, drop_epoch = -1;
  bool push = false, single = false;
  uint64_t seed = 1, budget_us = 200000;
};

struct Shared {
  Config cfg;
  std::vector<std::unique_ptr<Workspace>> ws;
  std::vector<ErrorWord> err;
  std::atomic<long long> mismatches{0};
  std::atomic<long long> timeouts{0};
};

inline uint32_t pattern(int rank, uint32_t epoch, int i) { return (uint32_t(rank) << 24) ^ (epoch * 2654435761u) ^ uint32_t(i); }

// st.release.sys into every rank's flag area (own copy included)
void signal_all(Shared& s, int rank, int slot, uint32_t epoch) {
  for (int p = 0; p < s.cfg.ranks; ++p) s.ws[p]->flags[slot * kMaxRanks + rank].store(epoch, std::memory_order_release);
}

// ld.acquire.sys poll of the own copy with a time budget; records the first failure like record_error()
bool wait_flag(Shared& s, int rank, int slot, int src, uint32_t epoch, uint32_t site) {
  const auto t0 = std::chrono::steady_clock::now();
  for (uint32_t spin = 0;; ++spin) {
    const uint32_t v = s.ws[rank]->flags[slot * kMaxRanks + src].load(std::memory_order_acquire);
    if (int32_t(v - epoch) >= 0) return true;
    if ((spin & 0x3f) == 0x3f) {
      const auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
      if (uint64_t(us) > s.cfg.budget_us) {
        uint32_t expected = 0;
        if (s.err[rank].code.compare_exchange_strong(expected, (site << 16) | 2u)) {
          s.err[rank].site = site;
          s.err[rank].src = uint32_t(src);
          s.err[rank].epoch = epoch;
        }
        s.timeouts.fetch_add(1);
        return false;
      }
      std::this_thread::yield();
    }
  }
}

void jitter(std::mt19937_64& rng) {
  const unsigned r = unsigned(rng() & 0xff);
  if (r < 96) std::this_thread::yield();
  if (r < 8) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
}

void run_rank(Shared& s, int rank) {
  const Config& c = s.cfg;
  std::mt19937_64 rng(c.seed * 1000003ull + uint64_t(rank));
  for (uint32_t e = 1; e <= uint32_t(c.epochs); ++e) {
    if (rank == c.drop_rank && int(e) == c.drop_epoch) return;       // leaves between steps, announcing nothing
    const int buf = c.single ? 0 : int(e & 1);
    jitter(rng);
    if (!c.push) {
      uint32_t* mine = s.ws[rank]->payload.data() + size_t(buf) * kBlock;
      for (int i = 0; i < kBlock; ++i) mine[i] = pattern(rank, e, i);
      signal_all(s, rank, kSlotData, e);
      for (int k = 1; k < c.ranks; ++k) {
        const int src = (rank + k) % c.ranks;
        if (!wait_flag(s, rank, kSlotData, src, e, 0x11)) return;   // a wait that gave up ends this rank's work
        jitter(rng);
        const uint32_t* theirs = s.ws[src]->payload.data() + size_t(buf) * kBlock;
        for (int i = 0; i < kBlock; ++i)
          if (theirs[i] != pattern(src, e, i)) {
            s.mismatches.fetch_add(1);
            break;
          }
      }
    } else {
      for (int k = 0; k < c.ranks; ++k) {                            // owners visited in an order rotated by rank
        const int owner = (rank + k) % c.ranks;
        uint32_t* slot = s.ws[owner]->payload.data() + (size_t(buf) * c.ranks + rank) * kBlock;
        for (int i = 0; i < kBlock; ++i) slot[i] = pattern(rank, e, i) + uint32_t(owner);
        jitter(rng);
      }
      signal_all(s, rank, kSlotData, e);
      for (int src = 0; src < c.ranks; ++src)
        if (!wait_flag(s, rank, kSlotData, src, e, 0x12)) return;
      jitter(rng);
      for (int i = 0; i < kBlock; ++i) {                              // the owner's slot reduction
        uint32_t sum = 0, want = 0;
        for (int src = 0; src < c.ranks; ++src) {
          sum += s.ws[rank]->payload[(size_t(buf) * c.ranks + src) * kBlock + i];
          want += pattern(src, e, i) + uint32_t(rank);
        }
        if (sum != want) {
          s.mismatches.fetch_add(1);
          break;
        }
      }
    }
  }
}

}  // namespace

int main(int argc, char** argv) {
  Shared s;
  Config& c = s.cfg;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : "0"; };
    if (a == "--ranks") c.ranks = std::atoi(next());
    else if (a == "--epochs") c.epochs = std::atoi(next());
    else if (a == "--seed") c.seed = std::strtoull(next(), nullptr, 10);
    else if (a == "--mode") c.push = std::string(next()) == "push";
    else if (a == "--single-buffer") c.single = true;
    else if (a == "--drop-rank") c.drop_rank = std::atoi(next());
    else if (a == "--drop-epoch") c.drop_epoch = std::atoi(next());
    else if (a == "--budget-us") c.budget_us = std::strtoull(next(), nullptr, 10);
    else { std::fprintf(stderr, "unknown flag %s\n", a.c_str()); return 2; }
  }
  if (c.ranks < 2 || c.ranks > kMaxRanks || c.epochs < 1) { std::fprintf(stderr, "ranks in [2, %d], epochs >= 1\n", kMaxRanks); return 2; }
  s.err = std::vector<ErrorWord>(c.ranks);
  for (int r = 0; r < c.ranks; ++r) {
    s.ws.emplace_back(new Workspace());
    for (auto& f : s.ws[r]->flags) f.store(0, std::memory_order_relaxed);
    s.ws[r]->payload.assign(size_t(2) * (c.push ? c.ranks : 1) * kBlock, 0u);
  }
  std::vector<std::thread> threads;
  for (int r = 0; r < c.ranks; ++r) threads.emplace_back(run_rank, std::ref(s), r);
  for (auto& t : threads) t.join();
  int first_err_rank = -1;
  for (int r = 0; r < c.ranks; ++r)
    if (s.err[r].code.load() != 0 && first_err_rank < 0) first_err_rank = r;
  std::printf("{\"mode\": \"%s\", \"ranks\": %d, \"epochs\": %d, \"single_buffer\": %s, \"mismatches\": %lld, \"timeouts\": %lld",
              c.push ? "push" : "pull", c.ranks, c.epochs, c.single ? "true" : "false", s.mismatches.load(), s.timeouts.load());
  if (first_err_rank >= 0)
    std::printf(", \"error\": {\"rank\": %d, \"site\": %u, \"src\": %u, \"epoch\": %u}", first_err_rank, s.err[first_err_rank].site,
                s.err[first_err_rank].src, s.err[first_err_rank].epoch);
  std::printf("}\n");
  return s.mismatches.load() == 0 ? 0 : 1;
}
