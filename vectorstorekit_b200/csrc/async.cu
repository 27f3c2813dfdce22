// The asynchronous form of a search: submit, return, be called back.
//
// The reference's engine is an actor whose batch call commits a command buffer and resumes a continuation from the
// buffer's completion handler (Acceleration/MetalAccelerationEngine.swift:139-204, :444-449; the same shape in
// Acceleration/Metal/MetalDistanceCompute.swift:365-375).  A search here is not one enqueue: the chunk schedule reads
// candidate counts back between launches and a query whose certificate fails is re-run, so a stream callback alone
// cannot carry it.  Each context therefore owns one worker thread.  vsk_search_async / vsk_search_dev_async put the
// blocking call on the worker's queue and return; the worker runs the calls in submission order on the context's
// stream and then calls `done(user, status)` from its own thread.  vsk_wait blocks until the queue is empty.
//
// Between a submission and its completion the context belongs to the worker: the caller makes no other call on the
// context or its indices except further *_async submissions, vsk_wait and vsk_last_error (after completion).
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace vsk {

struct Worker {
  std::thread th;
  std::mutex m;
  std::condition_variable wake, idle;
  std::deque<std::function<void()>> jobs;
  int running = 0;
  bool stop = false;
  int32_t first_failure = VSK_OK;   // first non-OK status since the last vsk_wait
};

namespace {

void worker_main(Ctx* ctx, Worker* w) {
  cudaSetDevice(ctx->device);
  for (;;) {
    std::function<void()> job;
    {
      std::unique_lock<std::mutex> lk(w->m);
      w->wake.wait(lk, [&] { return w->stop || !w->jobs.empty(); });
      if (w->jobs.empty()) return;   // stop requested and nothing left
      job = std::move(w->jobs.front());
      w->jobs.pop_front();
      w->running = 1;
    }
    job();
    {
      std::lock_guard<std::mutex> lk(w->m);
      w->running = 0;
      if (w->jobs.empty()) w->idle.notify_all();
    }
  }
}

Worker* worker_of(Ctx* ctx) {
  if (!ctx->worker) {
    ctx->worker = new Worker();
    ctx->worker->th = std::thread(worker_main, ctx, ctx->worker);
  }
  return ctx->worker;
}

int32_t submit(Ctx* ctx, std::function<int32_t()> call, vsk_done_fn done, void* user) {
  Worker* w = worker_of(ctx);
  {
    std::lock_guard<std::mutex> lk(w->m);
    w->jobs.emplace_back([w, call = std::move(call), done, user] {
      const int32_t st = call();
      if (st != VSK_OK) {
        std::lock_guard<std::mutex> lk2(w->m);
        if (w->first_failure == VSK_OK) w->first_failure = st;
      }
      if (done) done(user, st);
    });
  }
  w->wake.notify_one();
  return VSK_OK;
}

}  // namespace

// Drains the queue and joins the worker (vsk_close).
void worker_release(Ctx* ctx) {
  Worker* w = ctx->worker;
  if (!w) return;
  {
    std::lock_guard<std::mutex> lk(w->m);
    w->stop = true;
  }
  w->wake.notify_all();
  if (w->th.joinable()) w->th.join();
  delete w;
  ctx->worker = nullptr;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_search_async(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, float* out_dist,
                         int64_t* out_ids, vsk_done_fn done, void* user) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  return submit(ix->ctx, [=] { return vsk_search(i, q, nq, k, qmasks, out_dist, out_ids); }, done, user);
}

int32_t vsk_search_dev_async(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks,
                             float* out_dist, int64_t* out_ids, vsk_done_fn done, void* user) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  return submit(ctx, [=] {
    const int32_t st = vsk_search_dev(i, q, nq, k, qmasks, out_dist, out_ids);
    if (st != VSK_OK) return st;
    // the callback promises finished results: the device form ends with the stream drained
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess)
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "stream synchronisation failed after an asynchronous search");
    return (int32_t)VSK_OK;
  }, done, user);
}

int32_t vsk_wait(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  Worker* w = ctx->worker;
  if (!w) return VSK_OK;
  std::unique_lock<std::mutex> lk(w->m);
  w->idle.wait(lk, [&] { return w->jobs.empty() && !w->running; });
  const int32_t st = w->first_failure;
  w->first_failure = VSK_OK;
  return st;
}

}  // extern "C"
