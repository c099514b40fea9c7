// Range reader for safetensors shards: reads exactly the bytes a rank needs (whole tensors, row
// ranges, column ranges) with positional reads spread over a few threads, straight into a caller's
// buffer (a pinned host tensor in practice).  Plain C ABI, no torch and no CUDA, so it builds and is
// tested on machines without a GPU.  The header (8-byte little-endian length + JSON) is parsed by
// the Python side; this file only moves bytes.
//
// Counterpart in the reference: the rank-local streaming loader
// (crates/ferrl/src/sharded_safetensors.rs:644-750) which seeks to each tensor's byte range.
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

// Reads [off, off+n) fully; returns 0 or a negative errno (-EIO on a short file).
int pread_full(int fd, char* dst, uint64_t n, uint64_t off) {
  while (n > 0) {
    const size_t want = static_cast<size_t>(std::min<uint64_t>(n, 1ull << 30));
    const ssize_t got = ::pread(fd, dst, want, static_cast<off_t>(off));
    if (got < 0) {
      if (errno == EINTR) continue;
      return -errno;
    }
    if (got == 0) return -EIO;
    dst += got;
    off += static_cast<uint64_t>(got);
    n -= static_cast<uint64_t>(got);
  }
  return 0;
}

int clamp_threads(int threads, uint64_t work_items) {
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  int t = threads <= 0 ? static_cast<int>(std::min(8u, hw)) : threads;
  t = static_cast<int>(std::min<uint64_t>(static_cast<uint64_t>(t), std::max<uint64_t>(1, work_items)));
  return std::max(1, std::min(t, 64));
}

}  // namespace

extern "C" {

// Contiguous range -> dst.  Split into `threads` pieces of at least 4 MiB.
int ferrl_read_range(const char* path, uint64_t offset, uint64_t nbytes, void* dst, int threads) {
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return -errno;
  const uint64_t min_piece = 4ull << 20;
  const int t = clamp_threads(threads, (nbytes + min_piece - 1) / min_piece);
  std::atomic<int> status{0};
  auto work = [&](int i) {
    const uint64_t piece = (nbytes + t - 1) / t;
    const uint64_t lo = std::min<uint64_t>(nbytes, piece * i);
    const uint64_t hi = std::min<uint64_t>(nbytes, lo + piece);
    if (hi > lo) {
      const int rc = pread_full(fd, static_cast<char*>(dst) + lo, hi - lo, offset + lo);
      if (rc != 0) status.store(rc);
    }
  };
  if (t == 1) {
    work(0);
  } else {
    std::vector<std::thread> pool;
    for (int i = 0; i < t; ++i) pool.emplace_back(work, i);
    for (auto& th : pool) th.join();
  }
  ::close(fd);
  return status.load();
}

// `rows` pieces of `piece_bytes`, `src_stride` apart in the file, packed densely into dst: the
// column range [c0, c0+n) of a row-major matrix, or any other regular 2-D sub-block.
int ferrl_read_strided(const char* path, uint64_t offset, uint64_t src_stride, uint64_t rows, uint64_t piece_bytes,
                       void* dst, int threads) {
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return -errno;
  const int t = clamp_threads(threads, (rows + 255) / 256);
  std::atomic<int> status{0};
  auto work = [&](int i) {
    const uint64_t per = (rows + t - 1) / t;
    const uint64_t lo = std::min<uint64_t>(rows, per * i), hi = std::min<uint64_t>(rows, lo + per);
    for (uint64_t r = lo; r < hi; ++r) {
      const int rc = pread_full(fd, static_cast<char*>(dst) + r * piece_bytes, piece_bytes, offset + r * src_stride);
      if (rc != 0) {
        status.store(rc);
        return;
      }
    }
  };
  if (t == 1) {
    work(0);
  } else {
    std::vector<std::thread> pool;
    for (int i = 0; i < t; ++i) pool.emplace_back(work, i);
    for (auto& th : pool) th.join();
  }
  ::close(fd);
  return status.load();
}

// Header of a safetensors file: writes the JSON length to *json_len and copies at most `cap` bytes
// of the JSON text to `json`.  Returns 0, or a negative errno (-EINVAL for an implausible length).
int ferrl_read_header(const char* path, uint64_t* json_len, char* json, uint64_t cap) {
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return -errno;
  unsigned char len_le[8];
  int rc = pread_full(fd, reinterpret_cast<char*>(len_le), 8, 0);
  if (rc == 0) {
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | len_le[i];
    const off_t size = ::lseek(fd, 0, SEEK_END);
    if (size < 8 || n > static_cast<uint64_t>(size) - 8 || n > (1ull << 31)) {
      rc = -EINVAL;
    } else {
      *json_len = n;
      if (json != nullptr && cap > 0) rc = pread_full(fd, json, std::min(n, cap), 8);
    }
  }
  ::close(fd);
  return rc;
}

}  // extern "C"
