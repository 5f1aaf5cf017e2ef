// sanitize_main.cc — a native stress driver for the host runtime, built with -fsanitize=thread or
// -fsanitize=address (roc_shmem_b200/build.py: build_sanitizer_driver) and run by the CPU test suite.
// It exercises what host threads share: the buddy allocator, the team table, the CPU backend (PEs as threads
// over one shared mapping: puts, gets, atomics, waits, collectives, per-thread contexts) and the
// reverse-offload ring with several producers and a paused / resumed service thread.
// The reference has no sanitizer build; its host tests (clients/sos_tests: mt_contention.c, mt_a2a.c,
// threading.c) are the workloads repeated here.
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../include/bshmem.h"
#include "../include/bshmem_proxy.h"
#include "allocator.h"

using namespace bshmem;

#define CHECK(cond)                                                                  \
  do {                                                                               \
    if (!(cond)) {                                                                   \
      std::fprintf(stderr, "sanitize_main: check failed: %s (line %d)\n", #cond, __LINE__); \
      std::exit(1);                                                                  \
    }                                                                                \
  } while (0)

static void allocator_storm() {
  Pow2BuddyAllocator heap(8 << 20, 0, 128);
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t)
    ts.emplace_back([&heap, t] {
      std::vector<uint64_t> mine;
      for (int i = 0; i < 400; ++i) {
        uint64_t off = heap.alloc(128u << ((i + t) % 6));
        if (off != kNoOffset) mine.push_back(off);
        if (mine.size() > 8) { heap.free(mine.front()); mine.erase(mine.begin()); }
      }
      for (uint64_t o : mine) heap.free(o);
    });
  for (auto& t : ts) t.join();
  CHECK(heap.alloc(8 << 20) != kNoOffset);   // everything coalesced back
}

static void pe_body(void* world, int pe, int n_pes) {
  bshmem_handle_t h = nullptr;
  CHECK(bshmem_cpu_init(world, pe, nullptr, &h) == BSHMEM_OK);
  const int nxt = (pe + 1) % n_pes;
  long* buf = static_cast<long*>(bshmem_malloc(h, 1024 * sizeof(long)));
  unsigned long long* ctr = static_cast<unsigned long long*>(bshmem_calloc(h, 4, 8));
  long* red = static_cast<long*>(bshmem_malloc(h, 256 * sizeof(long)));
  CHECK(buf && ctr && red);
  // several host threads of one PE: shared default context and contexts of their own
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t)
    ts.emplace_back([=] {
      bshmem_ctx_t c = BSHMEM_CTX_INVALID;
      CHECK(bshmem_ctx_create(h, BSHMEM_CTX_SERIALIZED, &c) == BSHMEM_OK);
      long local[64];
      for (int i = 0; i < 64; ++i) local[i] = pe * 1000 + t * 100 + i;
      for (int rep = 0; rep < 20; ++rep) {
        CHECK(bshmem_ctx_putmem_nbi(h, c, buf + t * 64, local, sizeof(local), nxt) == BSHMEM_OK);
        CHECK(bshmem_ctx_quiet(h, c) == BSHMEM_OK);
        uint64_t old = 0;
        CHECK(bshmem_ctx_amo(h, BSHMEM_CTX_DEFAULT, BSHMEM_UINT64, BSHMEM_AMO_FETCH_ADD, ctr, 1, 0, nxt, &old) == BSHMEM_OK);
      }
      CHECK(bshmem_ctx_destroy(h, c) == BSHMEM_OK);
    });
  for (auto& t : ts) t.join();
  CHECK(bshmem_barrier_all(h) == BSHMEM_OK);
  CHECK(ctr[0] == 80ull);
  const int prv = (pe + n_pes - 1) % n_pes;
  for (int t = 0; t < 4; ++t) CHECK(buf[t * 64 + 5] == prv * 1000 + t * 100 + 5);
  for (int i = 0; i < 256; ++i) buf[i] = pe + i;
  CHECK(bshmem_barrier_all(h) == BSHMEM_OK);
  CHECK(bshmem_team_reduce(h, BSHMEM_TEAM_WORLD, BSHMEM_INT64, BSHMEM_SUM, red, buf, 256) == BSHMEM_OK);
  CHECK(red[3] == (long)(n_pes * 3 + n_pes * (n_pes - 1) / 2));
  // the ring: three producer threads, blocking and non-blocking commands
  bshmem_proxy_t* px = nullptr;
  CHECK(bshmem_proxy_create_host(h, 8, 2000000, &px) == BSHMEM_OK);
  std::vector<std::thread> prod;
  for (int t = 0; t < 3; ++t)
    prod.emplace_back([=] {
      for (int i = 0; i < 100; ++i) {
        bshmem_proxy_desc_t d;
        std::memset(&d, 0, sizeof(d));
        d.op = BSHMEM_PROXY_AMO; d.pe = nxt; d.dtype = BSHMEM_UINT64; d.sub_op = (i & 1) ? BSHMEM_AMO_ADD : BSHMEM_AMO_FETCH_ADD;
        d.sym_off = (uint64_t)(reinterpret_cast<char*>(ctr + 1) - static_cast<char*>(bshmem_heap_base(h)));
        d.value = 1;
        d.flags = (i & 1) ? 0 : BSHMEM_PROXY_FLAG_BLOCKING;
        uint64_t res = 0;
        CHECK(bshmem_proxy_host_submit(px, &d, &res) == BSHMEM_OK);
      }
    });
  for (auto& t : prod) t.join();
  bshmem_proxy_desc_t q;
  std::memset(&q, 0, sizeof(q));
  q.op = BSHMEM_PROXY_QUIET; q.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  CHECK(bshmem_proxy_host_submit(px, &q, nullptr) == BSHMEM_OK);
  CHECK(bshmem_proxy_stop(px) == BSHMEM_OK);
  CHECK(bshmem_barrier_all(h) == BSHMEM_OK);
  CHECK(ctr[1] == 300ull);
  bshmem_free(h, red);
  bshmem_free(h, ctr);
  bshmem_free(h, buf);
  CHECK(bshmem_finalize(h) == BSHMEM_OK);
}

int main() {
  allocator_storm();
  const int n_pes = 3;
  void* world = nullptr;
  std::string name = "/bshmem-sanitize-" + std::to_string((long)getpid());
  CHECK(bshmem_cpu_world_create(name.c_str(), n_pes, 4 << 20, &world) == BSHMEM_OK);
  std::vector<std::thread> pes;
  for (int p = 0; p < n_pes; ++p) pes.emplace_back(pe_body, world, p, n_pes);
  for (auto& t : pes) t.join();
  CHECK(bshmem_cpu_world_destroy(world) == BSHMEM_OK);
  std::puts("SANITIZE_OK");
  return 0;
}
