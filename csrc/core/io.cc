// File range reader for checkpoint loading: 64-bit offsets, strided 2-D slices (row and column partitions for
// tensor/expert parallel shards), several worker threads per call.  Returns 0 or a negative errno-style code.
// Counterpart of the reference's TP-partitioned range reads (rust/crates/ds41rt-loader/src/v41_catalog.rs:215-273).
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <thread>
#include <vector>

namespace {
int read_fully(int fd, uint8_t* dst, uint64_t n, uint64_t off) {
  while (n > 0) {
    const ssize_t r = pread(fd, dst, n > (1u << 30) ? (1u << 30) : n, static_cast<off_t>(off));
    if (r < 0) {
      if (errno == EINTR) continue;
      return -errno;
    }
    if (r == 0) return -EIO;      // truncated file
    dst += r;
    off += static_cast<uint64_t>(r);
    n -= static_cast<uint64_t>(r);
  }
  return 0;
}
}  // namespace

extern "C" {

long long ds41_file_size(const char* path) {
  struct stat st;
  if (stat(path, &st) != 0) return -errno;
  return static_cast<long long>(st.st_size);
}

// Read rows [row0, row1) x byte columns [col0, col1) of a row-major matrix with `row_bytes` per row that starts at
// `base` in the file, into a dense destination.
int ds41_read_slice(const char* path, uint64_t base, uint64_t row_bytes, uint64_t row0, uint64_t row1, uint64_t col0,
                    uint64_t col1, void* dst, int threads) {
  if (row1 < row0 || col1 < col0 || col1 > row_bytes) return -EINVAL;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return -errno;
  const uint64_t rows = row1 - row0, width = col1 - col0;
  uint8_t* out = static_cast<uint8_t*>(dst);
  int rc = 0;
  if (width == row_bytes) {
    // contiguous block: split by bytes
    const uint64_t total = rows * row_bytes;
    const int nt = threads < 1 ? 1 : (total < (8u << 20) ? 1 : threads);
    std::atomic<int> err{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) {
      const uint64_t a = total * t / nt, b = total * (t + 1) / nt;
      pool.emplace_back([=, &err] {
        const int r = read_fully(fd, out + a, b - a, base + row0 * row_bytes + a);
        if (r != 0) err.store(r);
      });
    }
    for (auto& th : pool) th.join();
    rc = err.load();
  } else {
    const int nt = threads < 1 ? 1 : (rows * width < (8u << 20) ? 1 : threads);
    std::atomic<int> err{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) {
      const uint64_t a = rows * t / nt, b = rows * (t + 1) / nt;
      pool.emplace_back([=, &err] {
        for (uint64_t r = a; r < b; ++r) {
          const int e = read_fully(fd, out + r * width, width, base + (row0 + r) * row_bytes + col0);
          if (e != 0) { err.store(e); return; }
        }
      });
    }
    for (auto& th : pool) th.join();
    rc = err.load();
  }
  close(fd);
  return rc;
}

}  // extern "C"
