// On-disk key -> fixed-size row store for embedding tables that do not fit in memory (the SSD tier behind the
// device / host caches of OneEmbedding). Rows are appended to a values file in blocks aligned to the
// device's physical block size and read / written with positioned I/O (O_DIRECT when the filesystem allows
// it, buffered otherwise); the key -> row-index map lives in memory.
//
// Snapshots are point-in-time: a snapshot is a copy of the index, and every row that exists when a snapshot is
// taken (or when the table is opened) is frozen from then on. Updating a key whose row is frozen appends a new
// row and re-points the index, so the rows a snapshot refers to keep their values; only rows written since the
// last snapshot are overwritten in place. Appends always go to the physical end of the values file, which never
// moves backwards, so loading an older snapshot and writing on cannot clobber rows of a younger one.
//
// Crash safety of the index: besides the full copy written by close() and by every snapshot, each put() appends
// its (key, row) pairs to `index.log` and flushes it; open() loads `index` and replays the log.
//
// Reference: oneflow/core/embedding/persistent_table.cpp (O_DIRECT + Linux AIO, :197-236, :395),
// persistent_table_key_value_store.cu.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "ofc_core.h"

namespace {

struct PTable {
  std::string dir;
  int value_bytes = 0, block_bytes = 512;
  int64_t row_stride = 0;  // value_bytes rounded up so that rows never straddle more blocks than needed
  int fd = -1;
  bool direct = false, read_only = false;
  std::unordered_map<int64_t, int64_t> index;  // key -> row number
  int64_t rows = 0;         // next row to append (physical end of the values file, in rows); never decreases
  int64_t frozen_rows = 0;  // rows below this number belong to a snapshot or an earlier session: never overwritten
  FILE* log = nullptr;      // index.log: (key, row) pairs appended by put()
  std::mutex mu;
  void* bounce = nullptr;  // block-aligned staging for O_DIRECT
  int64_t bounce_bytes = 0;

  int64_t aligned(int64_t n) const { return (n + block_bytes - 1) / block_bytes * block_bytes; }

  bool ensure_bounce(int64_t n) {
    if (n <= bounce_bytes) return true;
    std::free(bounce);
    bounce = nullptr;
    if (posix_memalign(&bounce, 4096, static_cast<size_t>(n)) != 0) return false;
    bounce_bytes = n;
    return true;
  }
  // Reads/writes the aligned window covering [off, off+len).
  bool io(bool write, int64_t off, void* data, int64_t len) {
    if (!direct) {
      ssize_t r = write ? ::pwrite(fd, data, static_cast<size_t>(len), off) : ::pread(fd, data, static_cast<size_t>(len), off);
      if (!write && r >= 0 && r < len) std::memset(static_cast<char*>(data) + r, 0, static_cast<size_t>(len - r));
      return r >= 0;
    }
    const int64_t a0 = off / block_bytes * block_bytes;
    const int64_t a1 = aligned(off + len);
    if (!ensure_bounce(a1 - a0)) return false;
    ssize_t r = ::pread(fd, bounce, static_cast<size_t>(a1 - a0), a0);
    if (r < 0) return false;
    if (r < a1 - a0) std::memset(static_cast<char*>(bounce) + r, 0, static_cast<size_t>(a1 - a0 - r));
    if (write) {
      std::memcpy(static_cast<char*>(bounce) + (off - a0), data, static_cast<size_t>(len));
      return ::pwrite(fd, bounce, static_cast<size_t>(a1 - a0), a0) == a1 - a0;
    }
    std::memcpy(data, static_cast<char*>(bounce) + (off - a0), static_cast<size_t>(len));
    return true;
  }
  bool save_index(const std::string& path) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return false;
    const int64_t n = static_cast<int64_t>(index.size());
    std::fwrite(&rows, sizeof(rows), 1, f);
    std::fwrite(&n, sizeof(n), 1, f);
    for (auto& kv : index) {
      std::fwrite(&kv.first, sizeof(int64_t), 1, f);
      std::fwrite(&kv.second, sizeof(int64_t), 1, f);
    }
    return std::fclose(f) == 0;
  }
  bool load_index(const std::string& path) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    int64_t n = 0, saved_rows = 0;
    bool ok = std::fread(&saved_rows, sizeof(saved_rows), 1, f) == 1 && std::fread(&n, sizeof(n), 1, f) == 1;
    if (ok && saved_rows > rows) rows = saved_rows;  // the append position only ever grows
    index.clear();
    index.reserve(static_cast<size_t>(n));
    for (int64_t i = 0; ok && i < n; ++i) {
      int64_t k, v;
      ok = std::fread(&k, sizeof(k), 1, f) == 1 && std::fread(&v, sizeof(v), 1, f) == 1;
      if (ok) index[k] = v;
    }
    std::fclose(f);
    return ok;
  }
};

}  // namespace

OFC_API void* ofc_ptable_open(const char* dir, int value_bytes, int block_bytes, int read_only) {
  if (value_bytes <= 0 || (block_bytes != 512 && block_bytes != 4096)) {
    ofc::fail("persistent table: value_bytes must be positive and block_bytes 512 or 4096");
    return nullptr;
  }
  ::mkdir(dir, 0755);
  std::string snaps = std::string(dir) + "/snapshots";
  ::mkdir(snaps.c_str(), 0755);
  auto* t = new PTable();
  t->dir = dir;
  t->value_bytes = value_bytes;
  t->block_bytes = block_bytes;
  t->row_stride = value_bytes;
  t->read_only = read_only != 0;
  const std::string vpath = t->dir + "/values";
  const int flags = (read_only ? O_RDONLY : (O_RDWR | O_CREAT));
  t->fd = ::open(vpath.c_str(), flags | O_DIRECT, 0644);
  t->direct = t->fd >= 0;
  if (t->fd < 0) t->fd = ::open(vpath.c_str(), flags, 0644);
  if (t->fd < 0) {
    ofc::fail("persistent table: cannot open " + vpath);
    delete t;
    return nullptr;
  }
  struct stat st;
  if (::fstat(t->fd, &st) == 0) t->rows = (st.st_size + t->row_stride - 1) / t->row_stride;
  t->load_index(t->dir + "/index");  // absent on first use
  const std::string lpath = t->dir + "/index.log";
  if (FILE* lf = std::fopen(lpath.c_str(), "rb")) {  // puts of a session that did not reach close()
    int64_t kv[2];
    while (std::fread(kv, sizeof(int64_t), 2, lf) == 2) {
      t->index[kv[0]] = kv[1];
      if (kv[1] >= t->rows) t->rows = kv[1] + 1;
    }
    std::fclose(lf);
  }
  t->frozen_rows = t->rows;
  if (!t->read_only) t->log = std::fopen(lpath.c_str(), "ab");
  return t;
}
OFC_API void ofc_ptable_close(void* p) {
  auto* t = static_cast<PTable*>(p);
  if (!t->read_only && t->save_index(t->dir + "/index")) {
    if (t->log) std::fclose(t->log);
    t->log = nullptr;
    ::unlink((t->dir + "/index.log").c_str());  // the full index now covers everything the log held
  }
  if (t->log) std::fclose(t->log);
  ::close(t->fd);
  std::free(t->bounce);
  delete t;
}
OFC_API int ofc_ptable_put(void* p, const int64_t* keys, const void* values, int64_t n) {
  auto* t = static_cast<PTable*>(p);
  if (t->read_only) return ofc::fail("persistent table: opened read-only");
  std::lock_guard<std::mutex> g(t->mu);
  const char* v = static_cast<const char*>(values);
  for (int64_t i = 0; i < n; ++i) {
    auto it = t->index.find(keys[i]);
    int64_t row;
    bool moved = true;
    if (it == t->index.end()) {
      row = t->rows++;
      t->index.emplace(keys[i], row);
    } else if (it->second < t->frozen_rows) {
      row = t->rows++;  // the old row belongs to a snapshot: leave it, append the new value
      it->second = row;
    } else {
      row = it->second;
      moved = false;
    }
    if (!t->io(true, row * t->row_stride, const_cast<char*>(v + i * t->value_bytes), t->value_bytes))
      return ofc::fail("persistent table: write failed");
    if (moved && t->log) {
      const int64_t kv[2] = {keys[i], row};
      std::fwrite(kv, sizeof(int64_t), 2, t->log);
    }
  }
  if (t->log) std::fflush(t->log);
  return 0;
}
OFC_API int64_t ofc_ptable_get(void* p, const int64_t* keys, void* values_out, uint8_t* found_out, int64_t n) {
  auto* t = static_cast<PTable*>(p);
  std::lock_guard<std::mutex> g(t->mu);
  char* out = static_cast<char*>(values_out);
  int64_t found = 0;
  for (int64_t i = 0; i < n; ++i) {
    auto it = t->index.find(keys[i]);
    if (it == t->index.end()) {
      std::memset(out + i * t->value_bytes, 0, static_cast<size_t>(t->value_bytes));
      if (found_out) found_out[i] = 0;
      continue;
    }
    if (!t->io(false, it->second * t->row_stride, out + i * t->value_bytes, t->value_bytes))
      return ofc::fail("persistent table: read failed");
    if (found_out) found_out[i] = 1;
    ++found;
  }
  return found;
}
OFC_API int64_t ofc_ptable_size(void* p) { return static_cast<int64_t>(static_cast<PTable*>(p)->index.size()); }
// Copies up to ``cap`` keys of the current index (unspecified order) into ``out``; returns how many were written.
OFC_API int64_t ofc_ptable_keys(void* p, int64_t* out, int64_t cap) {
  auto* t = static_cast<PTable*>(p);
  std::lock_guard<std::mutex> g(t->mu);
  int64_t n = 0;
  for (auto& kv : t->index) {
    if (n >= cap) break;
    out[n++] = kv.first;
  }
  return n;
}
OFC_API int ofc_ptable_save_snapshot(void* p, const char* name) {
  auto* t = static_cast<PTable*>(p);
  std::lock_guard<std::mutex> g(t->mu);
  ::fsync(t->fd);
  if (!t->save_index(t->dir + "/snapshots/" + name)) return ofc::fail("persistent table: cannot write the snapshot");
  t->frozen_rows = t->rows;  // every row written so far now belongs to this snapshot
  return 0;
}
OFC_API int ofc_ptable_load_snapshot(void* p, const char* name) {
  auto* t = static_cast<PTable*>(p);
  std::lock_guard<std::mutex> g(t->mu);
  if (!t->load_index(t->dir + "/snapshots/" + name)) return ofc::fail(std::string("persistent table: no snapshot named ") + name);
  t->frozen_rows = t->rows;
  return 0;
}
