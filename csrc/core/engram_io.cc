// Engram table I/O on the host: memory-mapped row tables, page-advice prefetch and a gather thread with a bounded set
// of staging slots.
//
// A table is a flat file of `rows` records of `row_bytes` bytes (256 e4m3 values + 8 UE8M0 scales = 264 bytes in the
// official layout).  A request names the hashed row ids of a pass; the gather thread copies those records into one
// staging slot (contiguous, in request order) while the GPU is busy with the layers before the Engram layer, and the
// owner uploads the slot when it reaches that layer.  Slots are a fixed pool: submit() refuses (-1) when none is free,
// so the producer can never run ahead of the consumer by more than the pool.  A pending request can be cancelled
// (speculative rows that were rejected); the thread checks the flag between records.
//
// Two measuring aids sit beside the pipeline.  ds41_engram_table_evict drops this one file's pages from the page cache
// (unmap-level advice, then file-level advice; nothing system-wide is touched) and ds41_engram_table_resident reports the
// fraction that is resident, so a cold-cache measurement can be set up and checked without privileges.
// ds41_engram_io_bench times the delivery of the records of synthetic passes (tokens x rows_per_token uniformly hashed
// ids, sorted and de-duplicated as the gather does) by four routes: page faults on the mapping, page advice followed by
// the copy, one pread per record, and preads spread over threads.
// Capability reference: scripts/native/bench-engram-io.cpp and scripts/native/drop-page-cache.c of the reference (the
// reference's dropper writes the system-wide drop_caches control; this one is scoped to the table's file);
// rust/crates/ds41rt-loader/src/mapped_rows.rs:15, engram_prefetch.rs:143, engram_gather.rs:126,
// engram_pipeline.rs:69 of the reference.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
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

// Drop the table's pages from the page cache.  0 = ok, -1 = bad handle, otherwise the errno-style code of the advice.
int ds41_engram_table_evict(void* table) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr) return -1;
  fsync(t->fd);                                                        // a freshly written file: dirty pages cannot be dropped
  if (madvise(t->map, t->bytes, MADV_DONTNEED) != 0) return 1;        // page-table entries of this mapping
  const int rc = posix_fadvise(t->fd, 0, 0, POSIX_FADV_DONTNEED);      // then the now unmapped cache pages
  madvise(t->map, t->bytes, MADV_RANDOM);
  return rc;
}

// Fraction of the table's pages that are in memory (-1 on error).
double ds41_engram_table_resident(void* table) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr) return -1.0;
  const size_t page = static_cast<size_t>(sysconf(_SC_PAGESIZE));
  const size_t n = (t->bytes + page - 1) / page;
  std::vector<unsigned char> vec(n);
  if (mincore(t->map, t->bytes, vec.data()) != 0) return -1.0;
  size_t in = 0;
  for (unsigned char v : vec) in += v & 1;
  return n ? static_cast<double>(in) / static_cast<double>(n) : 0.0;
}

// Time `iters` synthetic passes.  mode 0 = copy from the mapping (page faults on demand), 1 = page advice for every
// record, then the copy, 2 = one pread per record, 3 = preads over `threads` threads.  `evict_each` drops the table
// from the page cache before every pass (cold measurements).  out: {mean us, min us, max us, records per pass (mean),
// checksum}.  0 = ok, -1 = bad arguments, -2 = read error.
int ds41_engram_io_bench(void* table, int tokens, int rows_per_token, int mode, int threads, int iters, int evict_each,
                         uint64_t seed, double* out5) {
  Table* t = static_cast<Table*>(table);
  if (t == nullptr || tokens <= 0 || tokens > 65536 || rows_per_token <= 0 || rows_per_token > 256 || mode < 0 ||
      mode > 3 || iters <= 0 || threads <= 0 || threads > 64 || out5 == nullptr)
    return -1;
  const uint32_t rb = t->row_bytes;
  const long page = sysconf(_SC_PAGESIZE);
  std::vector<uint8_t> sink(static_cast<size_t>(tokens) * rows_per_token * rb);
  uint64_t state = seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull;
  auto next = [&state] {                                   // splitmix64
    uint64_t z = (state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  };
  double sum = 0, lo = 1e300, hi = 0, records = 0;
  uint64_t checksum = 0;
  std::atomic<int> failed{0};
  for (int it = 0; it < iters; ++it) {
    std::vector<uint64_t> ids(static_cast<size_t>(tokens) * rows_per_token);
    for (auto& id : ids) id = next() % t->rows;
    std::sort(ids.begin(), ids.end());
    ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
    if (evict_each) ds41_engram_table_evict(t);
    const auto t0 = std::chrono::steady_clock::now();
    if (mode == 0 || mode == 1) {
      if (mode == 1) {
        for (uint64_t id : ids) {
          const uint64_t off = id * rb, start = off / page * page;
          const uint64_t end = std::min<uint64_t>((off + rb + page - 1) / page * page, t->bytes);
          madvise(t->map + start, end - start, MADV_WILLNEED);
        }
      }
      for (size_t i = 0; i < ids.size(); ++i) std::memcpy(sink.data() + i * rb, t->map + ids[i] * rb, rb);
    } else {
      auto read_range = [&](size_t a, size_t b) {
        for (size_t i = a; i < b; ++i) {
          size_t done = 0;
          while (done < rb) {
            const ssize_t n = pread(t->fd, sink.data() + i * rb + done, rb - done, ids[i] * rb + done);
            if (n <= 0) { failed = 1; return; }
            done += static_cast<size_t>(n);
          }
        }
      };
      if (mode == 2 || threads == 1) {
        read_range(0, ids.size());
      } else {
        std::vector<std::thread> pool;
        const size_t per = (ids.size() + threads - 1) / threads;
        for (int w = 0; w < threads; ++w) {
          const size_t a = std::min(ids.size(), per * w), b = std::min(ids.size(), a + per);
          if (a < b) pool.emplace_back(read_range, a, b);
        }
        for (auto& th : pool) th.join();
      }
    }
    const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    if (failed) return -2;
    for (size_t i = 0; i < ids.size(); ++i) checksum += sink[i * rb] + sink[i * rb + rb - 1];
    sum += us;
    lo = std::min(lo, us);
    hi = std::max(hi, us);
    records += static_cast<double>(ids.size());
  }
  out5[0] = sum / iters;
  out5[1] = lo;
  out5[2] = hi;
  out5[3] = records / iters;
  out5[4] = static_cast<double>(checksum);
  return 0;
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
