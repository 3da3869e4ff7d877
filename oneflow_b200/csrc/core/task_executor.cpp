// Dependency-tracking instruction executor: instructions name the objects they read and write; an
// instruction becomes ready when every earlier instruction that conflicts with it (read-after-write,
// write-after-read, write-after-write on any object) has completed; ready instructions are handed to the
// worker thread of their stream, so independent streams overlap while each stream stays in order.
//
// This is the scheduling core of the reference's eager virtual machine (pending -> dependency DAG over
// Dependence objects -> ready -> dispatch to the stream's worker -> release;
// oneflow/core/vm/virtual_machine_engine.cpp:210-260, 426-458) with stream roles such as compute, h2d,
// d2h, collective and callback (oneflow/core/common/stream_type.h:25-35). The Python side uses it to run
// host callbacks, checkpoint writes and data-loader stages off the main thread in a defined order.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "ofc_core.h"

namespace {

struct Instr {
  ofc_task_fn fn;
  void* arg;
  int stream;
  std::atomic<int> pending{0};            // unfinished predecessors
  std::vector<std::shared_ptr<Instr>> successors;
  bool done = false;
};

struct ObjState {
  std::shared_ptr<Instr> last_writer;
  std::vector<std::shared_ptr<Instr>> readers_since_write;
};

struct StreamQ {
  std::deque<std::shared_ptr<Instr>> ready;
  std::mutex mu;
  std::condition_variable cv;
  std::thread th;
};

struct Executor {
  std::vector<std::unique_ptr<StreamQ>> streams;
  std::mutex graph_mu;  // protects objects / successors / done flags
  std::unordered_map<int64_t, ObjState> objects;
  std::vector<std::shared_ptr<Instr>> last_in_stream;  // a stream executes in submission order
  std::atomic<bool> stop{false};
  std::atomic<int64_t> submitted{0}, completed{0};
  std::mutex done_mu;
  std::condition_variable done_cv;

  void push_ready(const std::shared_ptr<Instr>& in) {
    StreamQ& q = *streams[static_cast<size_t>(in->stream)];
    {
      std::lock_guard<std::mutex> g(q.mu);
      q.ready.push_back(in);
    }
    q.cv.notify_one();
  }
  void worker(int s) {
    StreamQ& q = *streams[static_cast<size_t>(s)];
    while (true) {
      std::shared_ptr<Instr> in;
      {
        std::unique_lock<std::mutex> lk(q.mu);
        q.cv.wait(lk, [&] { return stop.load() || !q.ready.empty(); });
        if (q.ready.empty()) return;
        in = q.ready.front();
        q.ready.pop_front();
      }
      in->fn(in->arg);
      std::vector<std::shared_ptr<Instr>> wake;
      {
        std::lock_guard<std::mutex> g(graph_mu);
        in->done = true;
        for (auto& s2 : in->successors)
          if (s2->pending.fetch_sub(1) == 1) wake.push_back(s2);
        in->successors.clear();
      }
      for (auto& w : wake) push_ready(w);
      completed.fetch_add(1);
      {
        std::lock_guard<std::mutex> g(done_mu);
      }
      done_cv.notify_all();
    }
  }
};

void add_edge(const std::shared_ptr<Instr>& from, const std::shared_ptr<Instr>& to) {
  if (!from || from->done || from.get() == to.get()) return;
  for (auto& s : from->successors)
    if (s.get() == to.get()) return;
  from->successors.push_back(to);
  to->pending.fetch_add(1);
}

}  // namespace

OFC_API void* ofc_executor_create(int n_streams) {
  if (n_streams < 1 || n_streams > 64) {
    ofc::fail("executor: n_streams must be 1..64");
    return nullptr;
  }
  auto* e = new Executor();
  for (int i = 0; i < n_streams; ++i) e->streams.emplace_back(new StreamQ());
  e->last_in_stream.resize(static_cast<size_t>(n_streams));
  for (int i = 0; i < n_streams; ++i) e->streams[static_cast<size_t>(i)]->th = std::thread([e, i] { e->worker(i); });
  return e;
}
OFC_API void ofc_executor_destroy(void* p) {
  auto* e = static_cast<Executor*>(p);
  ofc_executor_wait_all(p, 60000);
  e->stop.store(true);
  for (auto& q : e->streams) {
    q->cv.notify_all();
    if (q->th.joinable()) q->th.join();
  }
  delete e;
}
OFC_API int ofc_executor_submit(void* p, int stream, ofc_task_fn fn, void* arg, const int64_t* reads, int n_reads,
                                const int64_t* writes, int n_writes) {
  auto* e = static_cast<Executor*>(p);
  if (stream < 0 || stream >= static_cast<int>(e->streams.size())) return ofc::fail("executor: bad stream index");
  auto in = std::make_shared<Instr>();
  in->fn = fn;
  in->arg = arg;
  in->stream = stream;
  in->pending.store(1);  // guard so that it cannot fire while edges are being added
  {
    std::lock_guard<std::mutex> g(e->graph_mu);
    add_edge(e->last_in_stream[static_cast<size_t>(stream)], in);
    e->last_in_stream[static_cast<size_t>(stream)] = in;
    for (int i = 0; i < n_reads; ++i) {
      ObjState& o = e->objects[reads[i]];
      add_edge(o.last_writer, in);  // read after write
      o.readers_since_write.push_back(in);
    }
    for (int i = 0; i < n_writes; ++i) {
      ObjState& o = e->objects[writes[i]];
      add_edge(o.last_writer, in);  // write after write
      for (auto& r : o.readers_since_write) add_edge(r, in);  // write after read
      o.readers_since_write.clear();
      o.last_writer = in;
    }
  }
  e->submitted.fetch_add(1);
  if (in->pending.fetch_sub(1) == 1) e->push_ready(in);
  return 0;
}
OFC_API int ofc_executor_wait_all(void* p, int timeout_ms) {
  auto* e = static_cast<Executor*>(p);
  std::unique_lock<std::mutex> lk(e->done_mu);
  const bool ok = e->done_cv.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                                      [&] { return e->completed.load() >= e->submitted.load(); });
  return ok ? 0 : ofc::fail("executor: timed out waiting for instructions to finish", -2);
}
OFC_API int64_t ofc_executor_completed(void* p) { return static_cast<Executor*>(p)->completed.load(); }
