// proxy.h — host side of reverse offload: the service thread that drains the
// command ring and executes each descriptor on behalf of the GPU (or of a host
// producer), and the executor interface that binds it to a transport.
//
// Parity: library/src/reverse_offload/backend_ro.cpp:246-259 (ro_net_poll),
// queue.cpp:52-62 (Queue::process), mpi_transport.cpp:82-255 (switch over command
// types).  The reference needs two CPU threads (poller + MPI progress engine with
// a mutex-protected std::queue between them); here the executor is synchronous, so
// one thread polls and executes.
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>
#include <thread>

#include "../include/bshmem.h"
#include "../include/bshmem_proxy.h"

namespace bshmem {

class ProxyExecutor {
 public:
  virtual ~ProxyExecutor() {}
  // Executes one command; *result receives the fetched value (G / fetching AMO).
  virtual int execute(const bshmem_proxy_desc_t& d, uint64_t* result) = 0;
  // Called once on the service thread before the first command (e.g. cudaSetDevice).
  virtual void thread_init() {}
};

// Executes commands through the runtime's own backend (CPU backend; also used when
// the producer is a host thread).
class RuntimeExecutor final : public ProxyExecutor {
 public:
  explicit RuntimeExecutor(bshmem_handle_t h) : h_(h) {}
  int execute(const bshmem_proxy_desc_t& d, uint64_t* result) override;
 private:
  bshmem_handle_t h_;
};

enum ProxyCounter { PX_PROCESSED = 0, PX_DROPPED, PX_IDLE_POLLS, PX_ERRORS, PX_RMA, PX_AMO, PX_COLL, PX_ORDER, PX_COUNT };

}  // namespace bshmem

struct bshmem_proxy {
  bshmem_proxy_ring_t ring{};
  std::unique_ptr<bshmem::ProxyExecutor> exec;
  std::thread worker;
  std::atomic<bool> stop{false}, paused{false};
  std::atomic<int> drop{0};
  std::atomic<uint64_t> counters[bshmem::PX_COUNT] = {};
  void (*free_ring)(bshmem_proxy*) = nullptr;   // releases the ring memory (malloc'd or pinned)
  void* ring_mem = nullptr;
  void* aux_mem = nullptr;
  std::atomic<unsigned long long> host_write_index{0};   // ticket counter when producers are host threads

  void run();
};

namespace bshmem {
// Carves slots / completion / result / read_index out of one zeroed block of
// proxy_ring_bytes(capacity) bytes and starts the service thread.
uint64_t proxy_ring_bytes(uint64_t capacity);
bshmem_proxy* proxy_start(void* zeroed_block, uint64_t capacity, unsigned long long* write_index,
                          unsigned long long timeout_ns, std::unique_ptr<ProxyExecutor> exec);
}
