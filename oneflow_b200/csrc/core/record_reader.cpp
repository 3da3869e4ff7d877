// Data readers: (1) length-prefixed record files (u64 length + payload, the framing of OFRecord files) read by
// a background thread into a bounded queue with an optional shuffle buffer; (2) memory-mapped token-bin
// datasets (a flat array of 2- or 4-byte token ids) from which [batch, seq+1] int64 samples are gathered —
// the GPT indexed-bin reader. Reference: oneflow/user/data/ofrecord_dataset.h, random_shuffle_dataset.h,
// gpt_dataset.cpp.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "common.h"
#include "ofc_core.h"

namespace {

struct Reader {
  FILE* f = nullptr;
  size_t prefetch = 8, shuffle = 0;
  std::mt19937_64 rng;
  std::deque<std::string> q;
  std::vector<std::string> pool;  // shuffle buffer
  std::mutex mu;
  std::condition_variable not_empty, not_full;
  std::thread th;
  bool eof = false, stop = false;
  int error = 0;          // set by the reader thread: -5 corrupt length prefix, -6 truncated record, -7 out of memory
  uint64_t file_bytes = 0, max_record = 0;

  void emit(std::string&& rec) {
    std::unique_lock<std::mutex> lk(mu);
    not_full.wait(lk, [&] { return stop || q.size() < prefetch; });
    if (stop) return;
    q.push_back(std::move(rec));
    not_empty.notify_one();
  }
  void run() {
    try {
      run_inner();
    } catch (...) {  // bad_alloc / length_error must not reach std::terminate from this thread
      std::lock_guard<std::mutex> g(mu);
      error = -7;
      eof = true;
      not_empty.notify_all();
    }
  }
  void fail_with(int code) {
    std::lock_guard<std::mutex> g(mu);
    error = code;
    eof = true;
    not_empty.notify_all();
  }
  void run_inner() {
    uint64_t pos = 0;
    while (true) {
      uint64_t len = 0;
      const size_t got = std::fread(&len, 1, sizeof(len), f);
      if (got == 0) break;                                   // clean end of data
      if (got != sizeof(len)) return fail_with(-6);          // the file ends inside a length prefix
      pos += sizeof(len);
      // the prefix is untrusted: it must fit in what is left of the file (and under the configured maximum)
      if (len > file_bytes - pos || (max_record && len > max_record)) return fail_with(-5);
      std::string rec(len, '\0');
      if (len && std::fread(&rec[0], 1, len, f) != len) return fail_with(-6);
      pos += len;
      if (shuffle > 1) {
        if (pool.size() < shuffle) {
          pool.push_back(std::move(rec));
          continue;
        }
        const size_t j = static_cast<size_t>(rng() % pool.size());
        std::swap(pool[j], rec);
      }
      emit(std::move(rec));
      {
        std::lock_guard<std::mutex> g(mu);
        if (stop) return;
      }
    }
    while (!pool.empty()) {
      const size_t j = static_cast<size_t>(rng() % pool.size());
      std::swap(pool[j], pool.back());
      emit(std::move(pool.back()));
      pool.pop_back();
    }
    std::lock_guard<std::mutex> g(mu);
    eof = true;
    not_empty.notify_all();
  }
};

struct Tokens {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t bytes = 0;
  int token_bytes = 2;
};

}  // namespace

OFC_API int ofc_records_write(const char* path, const void* const* records, const int64_t* lengths, int64_t n) {
  FILE* f = std::fopen(path, "wb");
  if (!f) return ofc::fail(std::string("records: cannot create ") + path);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t len = static_cast<uint64_t>(lengths[i]);
    std::fwrite(&len, sizeof(len), 1, f);
    if (len) std::fwrite(records[i], 1, len, f);
  }
  return std::fclose(f) == 0 ? 0 : ofc::fail("records: write failed");
}
OFC_API void* ofc_records_open(const char* path, int prefetch, int shuffle_buffer, uint64_t seed) {
  FILE* f = std::fopen(path, "rb");
  if (!f) {
    ofc::fail(std::string("records: cannot open ") + path);
    return nullptr;
  }
  auto* r = new Reader();
  r->f = f;
  if (std::fseek(f, 0, SEEK_END) == 0) {
    const long end = std::ftell(f);
    r->file_bytes = end > 0 ? static_cast<uint64_t>(end) : 0;
    std::fseek(f, 0, SEEK_SET);
  }
  if (const char* m = std::getenv("OFB_MAX_RECORD_BYTES")) r->max_record = std::strtoull(m, nullptr, 10);
  r->prefetch = static_cast<size_t>(prefetch > 0 ? prefetch : 8);
  r->shuffle = static_cast<size_t>(shuffle_buffer > 0 ? shuffle_buffer : 0);
  r->rng.seed(seed);
  r->th = std::thread([r] { r->run(); });
  return r;
}
OFC_API int64_t ofc_records_next(void* p, void* out, int64_t cap) {
  auto* r = static_cast<Reader*>(p);
  std::unique_lock<std::mutex> lk(r->mu);
  r->not_empty.wait(lk, [&] { return r->eof || !r->q.empty(); });
  if (r->q.empty()) {
    if (r->error == -5) return ofc::fail("records: corrupt length prefix (longer than the rest of the file)", -5);
    if (r->error == -6) return ofc::fail("records: the file ends inside a record", -6);
    if (r->error == -7) return ofc::fail("records: out of memory while reading a record", -7);
    return 0;
  }
  std::string& rec = r->q.front();
  if (static_cast<int64_t>(rec.size()) > cap) return ofc::fail("records: caller buffer too small", -3);
  const int64_t n = static_cast<int64_t>(rec.size());
  std::memcpy(out, rec.data(), rec.size());
  r->q.pop_front();
  r->not_full.notify_one();
  return n == 0 ? -4 : n;  // -4: an empty record (distinguished from end of data)
}
OFC_API void ofc_records_close(void* p) {
  auto* r = static_cast<Reader*>(p);
  {
    std::lock_guard<std::mutex> g(r->mu);
    r->stop = true;
  }
  r->not_full.notify_all();
  if (r->th.joinable()) r->th.join();
  std::fclose(r->f);
  delete r;
}

OFC_API void* ofc_tokens_open(const char* path, int token_bytes) {
  if (token_bytes != 2 && token_bytes != 4) {
    ofc::fail("tokens: token_bytes must be 2 or 4");
    return nullptr;
  }
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) {
    ofc::fail(std::string("tokens: cannot open ") + path);
    return nullptr;
  }
  struct stat st;
  fstat(fd, &st);
  void* m = st.st_size ? mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
  if (m == MAP_FAILED) {
    ::close(fd);
    ofc::fail("tokens: mmap failed");
    return nullptr;
  }
  auto* t = new Tokens();
  t->fd = fd;
  t->base = static_cast<const uint8_t*>(m);
  t->bytes = static_cast<size_t>(st.st_size);
  t->token_bytes = token_bytes;
  return t;
}
OFC_API int64_t ofc_tokens_count(void* p) {
  auto* t = static_cast<Tokens*>(p);
  return static_cast<int64_t>(t->bytes / static_cast<size_t>(t->token_bytes));
}
OFC_API int ofc_tokens_batch(void* p, const int64_t* sample_idx, int64_t batch, int64_t seq_len, int64_t stride, int64_t* out) {
  auto* t = static_cast<Tokens*>(p);
  const int64_t total = ofc_tokens_count(p);
  for (int64_t b = 0; b < batch; ++b) {
    const int64_t start = sample_idx[b] * stride;
    if (start < 0 || start + seq_len + 1 > total) return ofc::fail("tokens: sample index out of range");
    for (int64_t i = 0; i <= seq_len; ++i) {
      const uint8_t* src = t->base + (start + i) * t->token_bytes;
      out[b * (seq_len + 1) + i] = t->token_bytes == 2 ? *reinterpret_cast<const uint16_t*>(src)
                                                       : *reinterpret_cast<const uint32_t*>(src);
    }
  }
  return 0;
}
OFC_API void ofc_tokens_close(void* p) {
  auto* t = static_cast<Tokens*>(p);
  if (t->base) munmap(const_cast<uint8_t*>(t->base), t->bytes);
  ::close(t->fd);
  delete t;
}
