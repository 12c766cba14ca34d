// Native chunk I/O for sharded checkpoints (host only, no CUDA): many chunk files written or read at once by a pool of
// threads, each chunk carrying the zarr v3 `crc32c` codec's trailer (4 bytes, little endian, CRC-32C of the payload).
// Writes are atomic (temporary file + rename) and optionally fsync'ed.  Plays the part TensorStore plays under the
// reference's Orbax checkpointer (`olmax/checkpoint/utils.py:153-159`): getting many shards to disk in parallel outside
// the Python interpreter lock, and detecting damaged chunks when they are read back.
//
// C interface (loaded with ctypes from checkpoint/zarr3.py):
//   ob_crc32c(data, n)                                      CRC-32C (Castagnoli), hardware instruction when available
//   ob_ckpt_write_files(n, paths, ptrs, sizes, append_crc, do_fsync, n_threads)
//   ob_ckpt_read_files(n, paths, ptrs, sizes, has_crc, n_threads)   reads exactly sizes[i] payload bytes, verifies
//   ob_ckpt_last_error()                                     message of the first failure of the last call
// Both batch calls return 0, or 1 + index of the first file that failed.
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

#if defined(__SSE4_2__)
#include <nmmintrin.h>
#endif

namespace {

std::mutex g_err_mutex;
std::string g_err;

void set_error(const std::string& msg) {
  std::lock_guard<std::mutex> lock(g_err_mutex);
  if (g_err.empty()) g_err = msg;
}

uint32_t crc_table[8][256];
std::once_flag crc_once;

void init_crc_table() {
  const uint32_t poly = 0x82F63B78u;  // reflected Castagnoli polynomial
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ poly : c >> 1;
    crc_table[0][i] = c;
  }
  for (uint32_t i = 0; i < 256; ++i)
    for (int t = 1; t < 8; ++t) crc_table[t][i] = (crc_table[t - 1][i] >> 8) ^ crc_table[0][crc_table[t - 1][i] & 0xFF];
}

uint32_t crc32c_update(uint32_t crc, const uint8_t* p, size_t n) {
  crc = ~crc;
#if defined(__SSE4_2__)
  while (n && (reinterpret_cast<uintptr_t>(p) & 7)) {
    crc = _mm_crc32_u8(crc, *p++);
    --n;
  }
  uint64_t c = crc;
  while (n >= 8) {
    uint64_t v;
    std::memcpy(&v, p, 8);
    c = _mm_crc32_u64(c, v);
    p += 8;
    n -= 8;
  }
  crc = static_cast<uint32_t>(c);
  while (n--) crc = _mm_crc32_u8(crc, *p++);
#else
  std::call_once(crc_once, init_crc_table);
  while (n >= 8) {  // slicing-by-8
    uint32_t lo, hi;
    std::memcpy(&lo, p, 4);
    std::memcpy(&hi, p + 4, 4);
    lo ^= crc;
    crc = crc_table[7][lo & 0xFF] ^ crc_table[6][(lo >> 8) & 0xFF] ^ crc_table[5][(lo >> 16) & 0xFF] ^
          crc_table[4][lo >> 24] ^ crc_table[3][hi & 0xFF] ^ crc_table[2][(hi >> 8) & 0xFF] ^
          crc_table[1][(hi >> 16) & 0xFF] ^ crc_table[0][hi >> 24];
    p += 8;
    n -= 8;
  }
  while (n--) crc = (crc >> 8) ^ crc_table[0][(crc ^ *p++) & 0xFF];
#endif
  return ~crc;
}

bool write_all(int fd, const uint8_t* p, size_t n) {
  while (n) {
    const size_t want = n < (size_t(1) << 30) ? n : (size_t(1) << 30);
    const ssize_t w = ::write(fd, p, want);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

bool read_all(int fd, uint8_t* p, size_t n) {
  while (n) {
    const size_t want = n < (size_t(1) << 30) ? n : (size_t(1) << 30);
    const ssize_t r = ::read(fd, p, want);
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    if (r == 0) return false;  // short file
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool write_one(const char* path, const uint8_t* data, uint64_t size, int append_crc, int do_fsync) {
  const std::string tmp = std::string(path) + ".tmp" + std::to_string(::getpid());
  const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) {
    set_error(std::string("open ") + tmp + ": " + std::strerror(errno));
    return false;
  }
  bool ok = write_all(fd, data, size);
  if (ok && append_crc) {
    const uint32_t crc = crc32c_update(0, data, size);
    const uint8_t le[4] = {uint8_t(crc), uint8_t(crc >> 8), uint8_t(crc >> 16), uint8_t(crc >> 24)};
    ok = write_all(fd, le, 4);
  }
  if (ok && do_fsync) ok = ::fsync(fd) == 0;
  const int saved = errno;
  ::close(fd);
  if (!ok) {
    set_error(std::string("write ") + tmp + ": " + std::strerror(saved));
    ::unlink(tmp.c_str());
    return false;
  }
  if (::rename(tmp.c_str(), path) != 0) {
    set_error(std::string("rename to ") + path + ": " + std::strerror(errno));
    ::unlink(tmp.c_str());
    return false;
  }
  return true;
}

bool read_one(const char* path, uint8_t* data, uint64_t size, int has_crc) {
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) {
    set_error(std::string("open ") + path + ": " + std::strerror(errno));
    return false;
  }
  struct stat st;
  const uint64_t expect = size + (has_crc ? 4 : 0);
  if (::fstat(fd, &st) != 0 || static_cast<uint64_t>(st.st_size) != expect) {
    set_error(std::string("chunk ") + path + " has " + std::to_string(static_cast<long long>(st.st_size)) +
              " bytes, expected " + std::to_string(static_cast<unsigned long long>(expect)) +
              " (truncated or corrupt checkpoint)");
    ::close(fd);
    return false;
  }
  bool ok = read_all(fd, data, size);
  uint8_t le[4] = {0, 0, 0, 0};
  if (ok && has_crc) ok = read_all(fd, le, 4);
  ::close(fd);
  if (!ok) {
    set_error(std::string("read ") + path + " failed");
    return false;
  }
  if (has_crc) {
    const uint32_t stored = uint32_t(le[0]) | (uint32_t(le[1]) << 8) | (uint32_t(le[2]) << 16) | (uint32_t(le[3]) << 24);
    const uint32_t crc = crc32c_update(0, data, size);
    if (crc != stored) {
      char buf[96];
      std::snprintf(buf, sizeof buf, " checksum mismatch (stored %08x, computed %08x): corrupt checkpoint", stored, crc);
      set_error(std::string("chunk ") + path + buf);
      return false;
    }
  }
  return true;
}

template <typename F>
int run_pool(int n, int n_threads, F&& one) {
  {
    std::lock_guard<std::mutex> lock(g_err_mutex);
    g_err.clear();
  }
  if (n <= 0) return 0;
  if (n_threads <= 0) n_threads = 8;
  if (n_threads > n) n_threads = n;
  std::atomic<int> next{0};
  std::atomic<int> first_bad{-1};
  auto worker = [&]() {
    for (;;) {
      const int i = next.fetch_add(1);
      if (i >= n) return;
      if (!one(i)) {
        int expected = -1;
        first_bad.compare_exchange_strong(expected, i);
      }
    }
  };
  std::vector<std::thread> threads;
  for (int t = 1; t < n_threads; ++t) threads.emplace_back(worker);
  worker();
  for (auto& t : threads) t.join();
  return first_bad.load() < 0 ? 0 : 1 + first_bad.load();
}

}  // namespace

extern "C" {

uint32_t ob_crc32c(const void* data, uint64_t n) { return crc32c_update(0, static_cast<const uint8_t*>(data), n); }

int ob_ckpt_write_files(int n, const char* const* paths, const void* const* ptrs, const uint64_t* sizes, int append_crc,
                        int do_fsync, int n_threads) {
  return run_pool(n, n_threads, [&](int i) {
    return write_one(paths[i], static_cast<const uint8_t*>(ptrs[i]), sizes[i], append_crc, do_fsync);
  });
}

int ob_ckpt_read_files(int n, const char* const* paths, void* const* ptrs, const uint64_t* sizes, int has_crc,
                       int n_threads) {
  return run_pool(n, n_threads,
                  [&](int i) { return read_one(paths[i], static_cast<uint8_t*>(ptrs[i]), sizes[i], has_crc); });
}

const char* ob_ckpt_last_error() {
  static thread_local std::string copy;
  std::lock_guard<std::mutex> lock(g_err_mutex);
  copy = g_err;
  return copy.c_str();
}

}  // extern "C"
