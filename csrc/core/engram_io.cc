// Engram table I/O on the host: memory-mapped row tables, page-advice prefetch and a gather thread with a bounded set
// of staging slots.
//
// A table is a flat file of `rows` records of `row_bytes` bytes (256 e4m3 values + 8 UE8M0 scales = 264 bytes in the
// official layout).  A request names the hashed row ids of a pass; the gather thread copies those records into one
// staging slot (contiguous, in request order) while the GPU is busy with the layers before the Engram layer, and the
// owner uploads the slot when it reaches that layer.  Slots are a fixed pool: submit() refuses (-1) when none is free,
// so the producer can never run ahead of the consumer by more than the pool.  A pending request can be cancelled
// (speculative rows that were rejected); the thread checks the flag between records.
// Capability reference: rust/crates/ds41rt-loader/src/mapped_rows.rs:15, engram_prefetch.rs:143, engram_gather.rs:126,
// engram_pipeline.rs:69 of the reference.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct Table {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t bytes = 0;
  uint64_t rows = 0;
  uint32_t row_bytes = 0;
};

enum SlotState : int { kFree = 0, kQueued = 1, kRunning = 2, kReady = 3, kCancelled = 4, kFailed = 5 };

struct Slot {
  std::vector<uint64_t> ids;
  uint8_t* data = nullptr;
  std::atomic<int> state{kFree};
  std::atomic<bool> cancel{false};
};

struct Gather {
  Table* table = nullptr;
  int max_rows = 0;
  std::vector<Slot> slots;
  std::deque<int> queue;
  std::mutex mu;
  std::condition_variable cv;
  bool stop = false;
  std::thread worker;
  std::atomic<uint64_t> rows_copied{0}, requests{0}, refused{0}, cancelled{0};

  explicit Gather(int n) : slots(n) {}

  void run() {
    for (;;) {
      int s;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop || !queue.empty(); });
        if (stop && queue.empty()) return;
        s = queue.front();
        queue.pop_front();
      }
      Slot& slot = slots[s];
      int expect = kQueued;
      if (!slot.state.compare_exchange_strong(expect, kRunning)) continue;      // cancelled while queued
      const uint32_t rb = table->row_bytes;
      bool ok = true;
      for (size_t i = 0; i < slot.ids.size(); ++i) {
        if (slot.cancel.load(std::memory_order_relaxed)) { ok = false; break; }
        std::memcpy(slot.data + i * rb, table->map + slot.ids[i] * rb, rb);
      }
      if (ok) rows_copied += slot.ids.size();
      slot.state.store(ok ? kReady : kCancelled, std::memory_order_release);
    }
  }
};

}  // namespace

extern "C" {

void* ds41_engram_table_open(const char* path, uint64_t rows, uint32_t row_bytes, int* err) {
  auto fail = [&](int code) -> void* { if (err) *err = code; return nullptr; };
  if (path == nullptr || rows == 0 || row_bytes == 0) return fail(1);
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return fail(2);
  struct stat st;
  if (fstat(fd, &st) != 0 || static_cast<uint64_t>(st.st_size) != rows * row_bytes) {   // exact size, no trailing bytes
    ::close(fd);
    return fail(3);
  }
  void* map = mmap(nullptr, st.st_size, PROT_READ, MAP_SHARED, fd, 0);
  if (map == MAP_FAILED) {
    ::close(fd);
    return fail(4);
  }
  madvise(map, st.st_size, MADV_RANDOM);
  Table* t = new Table;
  t->fd = fd;
  t->map = static_cast<uint8_t*>(map);
  t->bytes = st.st_size;
  t->rows = rows;
  t->row_bytes = row_bytes;
  if (err) *err = 0;
  return t;
}

void ds41_engram_table_close(void* table) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr) return;
  munmap(t->map, t->bytes);
  ::close(t->fd);
  delete t;
}

// Ask the kernel to start reading the pages of these rows (known as soon as the token ids are known).
int ds41_engram_prefetch(void* table, const uint64_t* ids, int n) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr || ids == nullptr || n < 0) return -1;
  const long page = sysconf(_SC_PAGESIZE);
  int advised = 0;
  for (int i = 0; i < n; ++i) {
    if (ids[i] >= t->rows) return -2;
    const uint64_t off = ids[i] * t->row_bytes;
    const uint64_t start = off / page * page;
    const uint64_t end = (off + t->row_bytes + page - 1) / page * page;
    if (madvise(t->map + start, std::min<uint64_t>(end, t->bytes) - start, MADV_WILLNEED) == 0) ++advised;
  }
  return advised;
}

void* ds41_engram_gather_create(void* table, int n_slots, int max_rows) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr || n_slots <= 0 || n_slots > 64 || max_rows <= 0) return nullptr;
  Gather* g = new Gather(n_slots);
  g->table = t;
  g->max_rows = max_rows;
  for (auto& s : g->slots) {
    void* p = nullptr;
    if (posix_memalign(&p, 4096, static_cast<size_t>(max_rows) * t->row_bytes) != 0) {
      for (auto& q : g->slots) std::free(q.data);
      delete g;
      return nullptr;
    }
    s.data = static_cast<uint8_t*>(p);
  }
  g->worker = std::thread([g] { g->run(); });
  return g;
}

void ds41_engram_gather_destroy(void* gather) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr) return;
  {
    std::lock_guard<std::mutex> lk(g->mu);
    g->stop = true;
    for (auto& s : g->slots) s.cancel = true;
  }
  g->cv.notify_all();
  g->worker.join();
  for (auto& s : g->slots) std::free(s.data);
  delete g;
}

// Returns the slot (ticket) >= 0, -1 when every slot is in use, -2 for a bad id or size.
int ds41_engram_gather_submit(void* gather, const uint64_t* ids, int n) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || ids == nullptr || n <= 0 || n > g->max_rows) return -2;
  for (int i = 0; i < n; ++i)
    if (ids[i] >= g->table->rows) return -2;
  for (size_t s = 0; s < g->slots.size(); ++s) {
    int expect = kFree;
    if (g->slots[s].state.compare_exchange_strong(expect, kQueued)) {
      Slot& slot = g->slots[s];
      slot.ids.assign(ids, ids + n);
      slot.cancel = false;
      {
        std::lock_guard<std::mutex> lk(g->mu);
        g->queue.push_back(static_cast<int>(s));
      }
      ++g->requests;
      g->cv.notify_one();
      return static_cast<int>(s);
    }
  }
  ++g->refused;
  return -1;
}

// 1 ready, 0 pending, -1 cancelled, -2 bad ticket
int ds41_engram_gather_poll(void* gather, int ticket) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || ticket < 0 || ticket >= static_cast<int>(g->slots.size())) return -2;
  const int st = g->slots[ticket].state.load(std::memory_order_acquire);
  if (st == kReady) return 1;
  if (st == kCancelled) return -1;
  if (st == kFree) return -2;
  return 0;
}

const void* ds41_engram_gather_data(void* gather, int ticket) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || ticket < 0 || ticket >= static_cast<int>(g->slots.size())) return nullptr;
  return g->slots[ticket].state.load(std::memory_order_acquire) == kReady ? g->slots[ticket].data : nullptr;
}

void ds41_engram_gather_cancel(void* gather, int ticket) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || ticket < 0 || ticket >= static_cast<int>(g->slots.size())) return;
  Slot& s = g->slots[ticket];
  s.cancel = true;
  int expect = kQueued;
  if (s.state.compare_exchange_strong(expect, kCancelled)) ++g->cancelled;
}

// Give the slot back (after the upload, or after a cancelled request has been observed).
int ds41_engram_gather_release(void* gather, int ticket) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || ticket < 0 || ticket >= static_cast<int>(g->slots.size())) return -2;
  Slot& s = g->slots[ticket];
  const int st = s.state.load(std::memory_order_acquire);
  if (st != kReady && st != kCancelled) return -1;           // still queued or running
  s.state.store(kFree, std::memory_order_release);
  return 0;
}

void ds41_engram_gather_stats(void* gather, uint64_t* out4) {
  Gather* g = static_cast<Gather*>(gather);
  if (g == nullptr || out4 == nullptr) return;
  out4[0] = g->requests;
  out4[1] = g->rows_copied;
  out4[2] = g->refused;
  out4[3] = g->cancelled;
}

}  // extern "C"
