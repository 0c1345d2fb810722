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
//   zero : the three-flag protocol of the ZeRO engine's peer-memory path (parallel/zero.py, csrc/comm_kernels.cu:
//          gv_grad_reduce, gv_wait_zero, gv_adamw_push, gv_comm_wait_peers) on single-buffered gradient and parameter
//          buffers: READY(e) = my gradient bucket of step e is complete; every owner then reads its slice from all peers
//          and announces DONE(e) = I have finished reading; a rank overwrites its bucket for step e+1 only after every
//          peer's DONE(e) (zero_grad right after the step); every owner stores its updated parameter slice into every
//          peer's parameter buffer and announces PARAM(e), which the peers wait for before the next step reads the
//          parameters. `--clip` adds the job-wide all-reduce of the gradient norm (a barrier) between the two phases;
//          `--skip-done-wait` removes the DONE wait to show that the checker sees that hazard;
//
//   mailbox : the publish / pull transport of the context-parallel ring (parallel/fused.py::Mailbox): every rank
//          publishes a block per epoch into a buffer of parity e & 1 and pulls the blocks of SOME peers (the reader sets
//          are known to everybody); before reusing a buffer the writer waits only for the ranks that read its
//          publication e-2 to have announced e-1. `--skip-reader-wait` drops that wait (the hazard the checker must see);
//
// pull and push run with payload regions double buffered by epoch parity: a rank reuses the region of epoch e-2 at epoch e, which is safe
// because in epoch e-1 it waited for every peer's e-1 announcement, and a peer announces e-1 only after it finished
// with epoch e-2. `--single-buffer` removes the double buffering (one region for all epochs): readers then observe
// blocks of a later epoch, which the checker counts (this mode exists to show that the checker can see the hazard).
// Every wait is bounded, as on the device: `--drop-rank r --drop-epoch e` makes rank r stop at epoch e without
// announcing; the others' waits give up after the budget, record {site, src, epoch} and all threads still finish.
//
// The reference has no such tool (it has no in-kernel signalling at all).
//
//   g++ -std=c++17 -O1 -g -pthread [-fsanitize=thread] flag_protocol_sim.cpp -o flag_protocol_sim
//   ./flag_protocol_sim --ranks 4 --epochs 200 --mode pull|push|zero|mailbox [--seed S] [--single-buffer] [--clip] [--skip-done-wait] [--skip-reader-wait]
//                        [--drop-rank r --drop-epoch e]
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
constexpr int kSlotReady = 0, kSlotDone = 1, kSlotParam = 2;   // the ZeRO engine's slots

struct Workspace {
  std::atomic<uint32_t> flags[kSlots * kMaxRanks];
  std::vector<uint32_t> payload;   // pull: [2][kBlock]; push: [2][world][kBlock]; zero: gradients [world][kBlock] | parameters [world][kBlock]
};

struct ErrorWord {
  std::atomic<uint32_t> code{0};
  uint32_t site = 0, src = 0, epoch = 0;
};

struct Config {
  int ranks = 4, epochs = 100, drop_rank = -1, drop_epoch = -1;
  bool push = false, single = false, zero = false, skip_done = false, clip = false, mailbox = false, skip_reader = false;
  uint64_t seed = 1, budget_us = 200000;
};

struct Shared {
  Config cfg;
  std::vector<std::unique_ptr<Workspace>> ws;
  std::vector<ErrorWord> err;
  std::atomic<long long> mismatches{0};
  std::atomic<long long> timeouts{0};
  std::atomic<long long> arrived{0};     // zero mode: arrivals at the per-step barrier (stands for the job-wide all-reduce)
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

inline uint32_t grad_pattern(int rank, uint32_t epoch, int owner, int i) { return pattern(rank, epoch, i) + 977u * uint32_t(owner); }
inline uint32_t param_pattern(int owner, uint32_t epoch, int i) { return pattern(owner, epoch ^ 0x5a5a5a5au, i); }

// all ranks arrive before any leaves (bounded like every other wait)
bool step_barrier(Shared& s, int rank, uint32_t epoch) {
  s.arrived.fetch_add(1, std::memory_order_acq_rel);
  const long long want = static_cast<long long>(s.cfg.ranks) * epoch;
  const auto t0 = std::chrono::steady_clock::now();
  for (uint32_t spin = 0; s.arrived.load(std::memory_order_acquire) < want; ++spin) {
    if ((spin & 0x3f) == 0x3f) {
      const auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
      if (uint64_t(us) > s.cfg.budget_us) {
        uint32_t expected = 0;
        if (s.err[rank].code.compare_exchange_strong(expected, (0x16u << 16) | 2u)) {
          s.err[rank].site = 0x16;
          s.err[rank].src = 0;
          s.err[rank].epoch = epoch;
        }
        s.timeouts.fetch_add(1);
        return false;
      }
      std::this_thread::yield();
    }
  }
  return true;
}

// One training step of the ZeRO engine's peer-memory protocol per epoch.
void run_rank_zero(Shared& s, int rank) {
  const Config& c = s.cfg;
  std::mt19937_64 rng(c.seed * 1000003ull + uint64_t(rank));
  const size_t grad_off = 0, param_off = size_t(c.ranks) * kBlock;
  for (uint32_t e = 1; e <= uint32_t(c.epochs); ++e) {
    if (rank == c.drop_rank && int(e) == c.drop_epoch) return;
    jitter(rng);
    if (e > 1) {
      // forward / backward of this step read the parameters every owner pushed at the end of the previous step
      for (int src = 0; src < c.ranks; ++src) {
        if (!wait_flag(s, rank, kSlotParam, src, e - 1, 0x13)) return;
        const uint32_t* p = s.ws[rank]->payload.data() + param_off + size_t(src) * kBlock;
        for (int i = 0; i < kBlock; ++i)
          if (p[i] != param_pattern(src, e - 1, i)) {
            s.mismatches.fetch_add(1);
            break;
          }
      }
    }
    uint32_t* g = s.ws[rank]->payload.data() + grad_off;
    for (int owner = 0; owner < c.ranks; ++owner)
      for (int i = 0; i < kBlock; ++i) g[size_t(owner) * kBlock + i] = grad_pattern(rank, e, owner, i);
    signal_all(s, rank, kSlotReady, e);
    for (int k = 0; k < c.ranks; ++k) {                 // phase A: my slice of every rank's bucket
      const int src = (rank + k) % c.ranks;
      if (!wait_flag(s, rank, kSlotReady, src, e, 0x15)) return;
      jitter(rng);
      const uint32_t* theirs = s.ws[src]->payload.data() + grad_off + size_t(rank) * kBlock;
      for (int i = 0; i < kBlock; ++i)
        if (theirs[i] != grad_pattern(src, e, rank, i)) {
          s.mismatches.fetch_add(1);
          break;
        }
    }
    signal_all(s, rank, kSlotDone, e);
    // with gradient clipping the job-wide all-reduce of the norm sits here; without it nothing does
    if (c.clip && !step_barrier(s, rank, e)) return;
    jitter(rng);
    for (int k = 0; k < c.ranks; ++k) {                 // phase B: my updated slice into every rank's parameter buffer
      const int dst = (rank + k) % c.ranks;
      uint32_t* p = s.ws[dst]->payload.data() + param_off + size_t(rank) * kBlock;
      for (int i = 0; i < kBlock; ++i) p[i] = param_pattern(rank, e, i);
    }
    signal_all(s, rank, kSlotParam, e);
    // zero_grad right after the step: the peers read their slices of this bucket until they announce DONE(e)
    if (!c.skip_done)
      for (int src = 0; src < c.ranks; ++src)
        if (!wait_flag(s, rank, kSlotDone, src, e, 0x14)) return;
    for (size_t i = 0; i < size_t(c.ranks) * kBlock; ++i) g[i] = 0u;
  }
}

// does `reader` pull writer's publication of `epoch`? (a fixed pseudo-random relation every rank can evaluate)
inline bool reads(const Config& c, int reader, int writer, uint32_t epoch) {
  if (reader == writer) return false;
  uint64_t x = c.seed * 0x9E3779B97F4A7C15ull + uint64_t(reader) * 0xBF58476D1CE4E5B9ull + uint64_t(writer) * 0x94D049BB133111EBull + epoch;
  x ^= x >> 31; x *= 0xD6E8FEB86659FD93ull; x ^= x >> 29;
  return (x & 3u) != 0u;          // three quarters of the pairs
}

void run_rank_mailbox(Shared& s, int rank) {
  const Config& c = s.cfg;
  std::mt19937_64 rng(c.seed * 1000003ull + uint64_t(rank));
  for (uint32_t e = 1; e <= uint32_t(c.epochs); ++e) {
    if (rank == c.drop_rank && int(e) == c.drop_epoch) return;
    jitter(rng);
    const int buf = int(e & 1);
    if (e > 2 && !c.skip_reader)
      for (int r = 0; r < c.ranks; ++r)                      // exactly the readers of my publication e-2
        if (reads(c, r, rank, e - 2) && !wait_flag(s, rank, kSlotData, r, e - 1, 0x17)) return;
    uint32_t* mine = s.ws[rank]->payload.data() + size_t(buf) * kBlock;
    for (int i = 0; i < kBlock; ++i) mine[i] = pattern(rank, e, i);
    signal_all(s, rank, kSlotData, e);
    for (int k = 1; k < c.ranks; ++k) {
      const int src = (rank + k) % c.ranks;
      if (!reads(c, rank, src, e)) continue;
      if (!wait_flag(s, rank, kSlotData, src, e, 0x18)) return;
      jitter(rng);
      const uint32_t* theirs = s.ws[src]->payload.data() + size_t(buf) * kBlock;
      for (int i = 0; i < kBlock; ++i)
        if (theirs[i] != pattern(src, e, i)) {
          s.mismatches.fetch_add(1);
          break;
        }
    }
  }
}

void run_rank(Shared& s, int rank) {
  const Config& c = s.cfg;
  if (c.zero) return run_rank_zero(s, rank);
  if (c.mailbox) return run_rank_mailbox(s, rank);
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
    else if (a == "--mode") { const std::string m = next(); c.push = m == "push"; c.zero = m == "zero"; c.mailbox = m == "mailbox"; }
    else if (a == "--skip-reader-wait") c.skip_reader = true;
    else if (a == "--skip-done-wait") c.skip_done = true;
    else if (a == "--clip") c.clip = true;
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
    s.ws[r]->payload.assign(size_t(2) * ((c.push || c.zero) ? c.ranks : 1) * kBlock, 0u);
  }
  std::vector<std::thread> threads;
  for (int r = 0; r < c.ranks; ++r) threads.emplace_back(run_rank, std::ref(s), r);
  for (auto& t : threads) t.join();
  int first_err_rank = -1;
  for (int r = 0; r < c.ranks; ++r)
    if (s.err[r].code.load() != 0 && first_err_rank < 0) first_err_rank = r;
  std::printf("{\"mode\": \"%s\", \"ranks\": %d, \"epochs\": %d, \"single_buffer\": %s, \"mismatches\": %lld, \"timeouts\": %lld",
              c.zero ? "zero" : (c.mailbox ? "mailbox" : (c.push ? "push" : "pull")), c.ranks, c.epochs, c.single ? "true" : "false", s.mismatches.load(), s.timeouts.load());
  if (first_err_rank >= 0)
    std::printf(", \"error\": {\"rank\": %d, \"site\": %u, \"src\": %u, \"epoch\": %u}", first_err_rank, s.err[first_err_rank].site,
                s.err[first_err_rank].src, s.err[first_err_rank].epoch);
  std::printf("}\n");
  return s.mismatches.load() == 0 ? 0 : 1;
}
