// TEST INFRASTRUCTURE ONLY. Part of the CPU oracle: a C++ restatement of the reference CPU
// plugin, used by tests, the smoke check and the benchmark's CPU-baseline leg as the checker.
// Nothing in the shipped plugin links, loads or calls this.
//
// Thread pool with fixed task sizes and dynamic claiming, after plugins/cpu/src/pool.rs:131-176
// (`run_tasks`, `for_chunks`). What matters for parity is only that work is cut into chunks that do
// not depend on the thread count (pool.rs:17-19); how threads wait is a performance detail.
// PYTORCHES_CPU_THREADS sets the thread count (default: all logical cores, pool.rs:61-63).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace cpuref {

class Pool {
  public:
    static Pool &get() {
        static Pool *p = new Pool();  // leaked on purpose: workers outlive static destructors
        return *p;
    }
    size_t threads() const { return threads_; }

    // Runs f(t) for t in [0, tasks); returns when all are done. The caller works too.
    template <class F> void run_tasks(size_t tasks, const F &f) {
        if (tasks <= 1 || threads_ == 1) {
            for (size_t t = 0; t < tasks; ++t) f(t);
            return;
        }
        std::unique_lock<std::mutex> submit(submit_, std::try_to_lock);
        if (!submit.owns_lock()) {  // pool busy with another caller: run inline (pool.rs:140-147)
            for (size_t t = 0; t < tasks; ++t) f(t);
            return;
        }
        std::function<void(size_t)> fn = [&f](size_t t) { f(t); };
        {
            std::lock_guard<std::mutex> g(m_);
            job_ = &fn;
            n_ = tasks;
            next_.store(0, std::memory_order_relaxed);
            done_.store(0, std::memory_order_relaxed);
            ++epoch_;
        }
        cv_.notify_all();
        drain(fn, tasks);
        while (done_.load(std::memory_order_acquire) < tasks) std::this_thread::yield();
        {
            std::lock_guard<std::mutex> g(m_);
            job_ = nullptr;
        }
        // Wait until no worker still holds a pointer to `fn`.
        while (active_.load(std::memory_order_acquire) != 0) std::this_thread::yield();
    }

    // Splits [0, n) into chunks of `chunk` and runs f(lo, hi) on each (pool.rs:173-176).
    template <class F> void for_chunks(size_t n, size_t chunk, const F &f) {
        if (chunk == 0) chunk = 1;
        size_t tasks = (n + chunk - 1) / chunk;
        run_tasks(tasks, [&](size_t t) {
            size_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
            f(lo, hi);
        });
    }

  private:
    Pool() {
        size_t n = 0;
        if (const char *e = std::getenv("PYTORCHES_CPU_THREADS")) n = std::strtoul(e, nullptr, 10);
        if (n == 0) n = std::thread::hardware_concurrency();
        if (n == 0) n = 1;
        threads_ = n;
        for (size_t i = 1; i < n; ++i) std::thread([this] { worker(); }).detach();
    }

    void drain(const std::function<void(size_t)> &fn, size_t n) {
        for (;;) {
            size_t t = next_.fetch_add(1, std::memory_order_acq_rel);
            if (t >= n) return;
            fn(t);
            done_.fetch_add(1, std::memory_order_release);
        }
    }

    void worker() {
        unsigned long seen = 0;
        for (;;) {
            const std::function<void(size_t)> *fn;
            size_t n;
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [&] { return epoch_ != seen && job_ != nullptr; });
                seen = epoch_;
                fn = job_;
                n = n_;
                active_.fetch_add(1, std::memory_order_acq_rel);
            }
            drain(*fn, n);
            active_.fetch_sub(1, std::memory_order_acq_rel);
        }
    }

    size_t threads_ = 1;
    std::mutex submit_, m_;
    std::condition_variable cv_;
    const std::function<void(size_t)> *job_ = nullptr;
    size_t n_ = 0;
    unsigned long epoch_ = 0;
    std::atomic<size_t> next_{0}, done_{0}, active_{0};
};

}  // namespace cpuref
