// Multi-threaded self-test of the host runtime (libofb_core sources compiled in), meant to run under ThreadSanitizer and
// AddressSanitizer + UBSan: `python -m oneflow_b200.build --sanitizers` builds lib/ofb_core_selftest_{tsan,asan}, the test
// suite runs both and fails on any sanitizer report. What it drives:
//   * task_executor: a dependency chain through 4 streams over one plain (non-atomic) counter. The only thing that orders
//     the increments is the executor's read/write tracking, so a missing happens-before edge is a data race TSan reports;
//     plus independent tasks on all streams and a fan-in.
//   * bin_allocator: threads allocating, filling, checking and freeing blocks of mixed sizes concurrently.
//   * control_store: one server, client threads doing add / set / get / compare-set / barrier, heartbeats running.
//   * persistent_table: puts and gets from several threads, snapshots in between.
//   * record_reader: a file of records read through the background prefetch thread.
// Reference counterpart: the reference builds its runtime with -fsanitize options in CI (cmake/oneflow.cmake, BUILD_TYPE
// with sanitizers) and runs its C++ unit tests under them.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../ofc_core.h"

static int g_fail = 0;
#define CHECK(c)                                                              \
  do {                                                                        \
    if (!(c)) {                                                               \
      std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #c); \
      ++g_fail;                                                               \
    }                                                                         \
  } while (0)

static long long g_counter = 0;          // deliberately not atomic
static long long g_side[4] = {0, 0, 0, 0};
static void bump(void*) { ++g_counter; }
static void bump_side(void* p) { ++*static_cast<long long*>(p); }

static void test_executor() {
  void* e = ofc_executor_create(4);
  CHECK(e != nullptr);
  const int64_t obj = 1;
  const int n = 2000;
  for (int i = 0; i < n; ++i) CHECK(ofc_executor_submit(e, i % 4, bump, nullptr, nullptr, 0, &obj, 1) == 0);   // WAW chain across streams
  for (int s = 0; s < 4; ++s)
    for (int i = 0; i < 500; ++i) {
      const int64_t own = 100 + s;
      CHECK(ofc_executor_submit(e, s, bump_side, &g_side[s], nullptr, 0, &own, 1) == 0);
    }
  // fan-in: one task reads all four side objects and the chain object, then writes the chain object
  const int64_t reads[4] = {100, 101, 102, 103};
  CHECK(ofc_executor_submit(e, 2, bump, nullptr, reads, 4, &obj, 1) == 0);
  CHECK(ofc_executor_wait_all(e, 60000) == 0);
  CHECK(g_counter == n + 1);
  for (int s = 0; s < 4; ++s) CHECK(g_side[s] == 500);
  CHECK(ofc_executor_completed(e) == n + 2000 + 1);
  ofc_executor_destroy(e);
}

static void test_allocator() {
  void* a = ofc_allocator_create(0, 1 << 20);
  CHECK(a != nullptr);
  std::vector<std::thread> th;
  for (int t = 0; t < 4; ++t)
    th.emplace_back([a, t] {
      unsigned seed = 17u * (t + 1);
      std::vector<std::pair<unsigned char*, int>> live;
      for (int i = 0; i < 3000; ++i) {
        seed = seed * 1664525u + 1013904223u;
        if (live.size() < 32 && (seed >> 16) % 3 != 0) {
          const int bytes = 64 + static_cast<int>((seed >> 8) % 20000);
          auto* p = static_cast<unsigned char*>(ofc_allocator_alloc(a, bytes));
          if (!p) { ++g_fail; continue; }
          std::memset(p, t + 1, static_cast<size_t>(bytes));
          live.emplace_back(p, bytes);
        } else if (!live.empty()) {
          auto [p, bytes] = live.back();
          live.pop_back();
          for (int k = 0; k < bytes; k += 997)
            if (p[k] != t + 1) ++g_fail;          // somebody else wrote into a live block
          if (ofc_allocator_free(a, p) != 0) ++g_fail;
        }
      }
      for (auto& [p, bytes] : live) ofc_allocator_free(a, p);
    });
  for (auto& x : th) x.join();
  int64_t reserved = 0, in_use = 0, chunks = 0, free_blocks = 0;
  ofc_allocator_stats(a, &reserved, &in_use, &chunks, &free_blocks);
  CHECK(in_use == 0);
  CHECK(ofc_allocator_shrink(a) >= 1);
  ofc_allocator_destroy(a);
}

static void test_store() {
  const int world = 4;
  void* srv = ofc_store_server_start(0, world);
  CHECK(srv != nullptr);
  const int port = ofc_store_server_port(srv);
  std::atomic<long long> last_add{0};
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r)
    th.emplace_back([&, r] {
      void* c = ofc_store_client_connect("127.0.0.1", port, r, 10000);
      if (!c) { ++g_fail; return; }
      ofc_store_heartbeat_start(c, 20);
      for (int i = 0; i < 200; ++i) {
        const long long v = ofc_store_add(c, "counter", 1);
        long long prev = last_add.load();
        while (v > prev && !last_add.compare_exchange_weak(prev, v)) {}
      }
      const std::string key = "rank" + std::to_string(r);
      const std::string val = "value-of-" + std::to_string(r);
      if (ofc_store_set(c, key.c_str(), val.data(), static_cast<int>(val.size())) != 0) ++g_fail;
      if (ofc_store_barrier(c, "b1", world, 10000) != 0) ++g_fail;
      char buf[64];
      const std::string other = "rank" + std::to_string((r + 1) % world);
      const int len = ofc_store_get(c, other.c_str(), buf, sizeof(buf), 5000);
      if (len != static_cast<int>(val.size())) ++g_fail;
      // exactly one rank wins the compare-and-set
      const char* want = "owner";
      char out[16];
      const std::string me = std::to_string(r);
      ofc_store_compare_set(c, "cas", "", 0, me.data(), static_cast<int>(me.size()), out, sizeof(out));
      (void)want;
      if (ofc_store_barrier(c, "b2", world, 10000) != 0) ++g_fail;
      int lost[8];
      if (ofc_store_lost_ranks(c, 5000, lost, 8) != 0) ++g_fail;
      ofc_store_client_close(c);
    });
  for (auto& x : th) x.join();
  CHECK(last_add.load() == 200 * world);
  ofc_store_server_stop(srv);
}

static void test_table(const std::string& dir) {
  void* t = ofc_ptable_open(dir.c_str(), 32, 512, 0);
  CHECK(t != nullptr);
  std::vector<std::thread> th;
  for (int w = 0; w < 3; ++w)
    th.emplace_back([t, w] {
      for (int i = 0; i < 300; ++i) {
        int64_t keys[4];
        float vals[4][8];
        for (int k = 0; k < 4; ++k) {
          keys[k] = w * 100000 + i * 4 + k;
          for (int j = 0; j < 8; ++j) vals[k][j] = static_cast<float>(keys[k]) + j;
        }
        if (ofc_ptable_put(t, keys, vals, 4) != 0) ++g_fail;
        float back[4][8];
        uint8_t found[4];
        if (ofc_ptable_get(t, keys, back, found, 4) != 4) ++g_fail;
        for (int k = 0; k < 4; ++k)
          if (!found[k] || back[k][3] != static_cast<float>(keys[k]) + 3) ++g_fail;
        if (w == 0 && i % 100 == 50) ofc_ptable_save_snapshot(t, ("s" + std::to_string(i)).c_str());
      }
    });
  for (auto& x : th) x.join();
  CHECK(ofc_ptable_size(t) == 3 * 300 * 4);
  ofc_ptable_close(t);
}

static void test_records(const std::string& path) {
  const int n = 500;
  std::vector<std::string> recs;
  for (int i = 0; i < n; ++i) recs.push_back(std::string(static_cast<size_t>(10 + i % 90), static_cast<char>('a' + i % 26)));
  std::vector<const void*> ptrs;
  std::vector<int64_t> lens;
  for (auto& r : recs) {
    ptrs.push_back(r.data());
    lens.push_back(static_cast<int64_t>(r.size()));
  }
  CHECK(ofc_records_write(path.c_str(), ptrs.data(), lens.data(), n) == 0);
  void* r = ofc_records_open(path.c_str(), 16, 0, 1);
  CHECK(r != nullptr);
  char buf[256];
  int count = 0;
  while (true) {
    const int64_t len = ofc_records_next(r, buf, sizeof(buf));
    if (len <= 0) break;
    CHECK(len == lens[static_cast<size_t>(count)] && buf[0] == recs[static_cast<size_t>(count)][0]);
    ++count;
  }
  CHECK(count == n);
  ofc_records_close(r);
}

int main(int argc, char** argv) {
  const std::string tmp = argc > 1 ? argv[1] : "/tmp/ofb_selftest";
  std::string cmd = "mkdir -p " + tmp + "/table";
  if (std::system(cmd.c_str()) != 0) return 2;
  test_executor();
  test_allocator();
  test_store();
  test_table(tmp + "/table");
  test_records(tmp + "/records.bin");
  if (g_fail) {
    std::fprintf(stderr, "core selftest: %d failures\n", g_fail);
    return 1;
  }
  std::printf("core selftest ok\n");
  return 0;
}
