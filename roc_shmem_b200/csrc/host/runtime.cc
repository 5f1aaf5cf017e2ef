// runtime.cc — implementation of the host C API over a Backend.  See runtime.h.
#include "runtime.h"

#include <cstdio>
#include <cstring>

using namespace bshmem;

namespace {
thread_local bshmem_handle_t tls_current = nullptr;

const char* kStatNames[ST_COUNT] = {
    "put", "put_nbi", "get", "get_nbi", "put_signal", "p", "g",
    "amo_fetch_add", "amo_fetch_inc", "amo_fetch", "amo_fetch_cswap", "amo_add", "amo_inc", "amo_cswap",
    "amo_set", "amo_swap", "amo_fetch_and", "amo_fetch_or", "amo_fetch_xor", "amo_and", "amo_or", "amo_xor",
    "fence", "quiet", "wait_until", "test", "barrier_all", "sync_all", "team_sync",
    "broadcast", "to_all", "reduce_scatter", "fcollect", "alltoall",
    "malloc", "free", "ctx_create", "ctx_destroy", "team_split", "team_destroy",
    "bytes_put", "bytes_get", "timeouts"};

const int kAmoStat[BSHMEM_AMO_COUNT] = {
    ST_AMO_FADD, ST_AMO_FINC, ST_AMO_FETCH, ST_AMO_FCSWAP, ST_AMO_ADD, ST_AMO_INC, ST_AMO_CSWAP, ST_AMO_SET,
    ST_AMO_SWAP, ST_AMO_FAND, ST_AMO_FOR, ST_AMO_FXOR, ST_AMO_AND, ST_AMO_OR, ST_AMO_XOR};

inline bool valid_handle(bshmem_handle_t h) { return h && !h->finalized; }
}  // namespace

const char* bshmem::host_stat_name(int idx) { return (idx >= 0 && idx < ST_COUNT) ? kStatNames[idx] : "?"; }

bshmem_runtime::bshmem_runtime(std::unique_ptr<Backend> be, const bshmem_config_t& c) : cfg(c), backend(std::move(be)) {
  heap.reset(new Pow2BuddyAllocator(backend->heap_bytes(), backend->reserved_bytes(), BSHMEM_ALIGNMENT));
  teams.reset(new TeamTracker(backend->n_pes(), backend->my_pe(), cfg.max_teams));
  ctxs.resize(cfg.max_ctxs);
  ctxs[0].reset(new HostContext());
  ctxs[0]->live = true;
  ctxs[0]->stats.enable(cfg.profile != 0);
  global_stats.enable(cfg.profile != 0);
  backend->set_timeout_us(cfg.timeout_us);
}

bool bshmem_runtime::to_offset(const void* p, uint64_t n, uint64_t* off) const {
  const char* base = backend->local_base();
  const char* q = static_cast<const char*>(p);
  if (!p || q < base) return false;
  uint64_t o = (uint64_t)(q - base);
  if (o > backend->heap_bytes() || n > backend->heap_bytes() - o) return false;
  *off = o;
  return true;
}

int bshmem_runtime::fail(int code, const std::string& msg) {
  std::lock_guard<std::mutex> g(mu);
  last_error = msg;
  if (cfg.debug) fprintf(stderr, "[bshmem pe %d] error %d: %s\n", backend->my_pe(), code, msg.c_str());
  return code;
}

HostContext* bshmem_runtime::ctx(int idx) {
  if (idx < 0 || idx >= (int)ctxs.size() || !ctxs[idx] || !ctxs[idx]->live) return nullptr;
  HostContext* c = ctxs[idx].get();
  // PRIVATE: "used only by the thread that created it" (OpenSHMEM 1.5, 9.4.1).  Using it from another thread is a
  // program error; with debug checks on, the call is refused instead of racing on the context's state.
  if (cfg.debug && (c->options & BSHMEM_CTX_PRIVATE) && c->owner != std::this_thread::get_id()) {
    fail(BSHMEM_ERR_STATE, "a PRIVATE context was used by a thread that did not create it");
    return nullptr;
  }
  return c;
}

int bshmem_runtime::resolve_pe(int ctx_idx, int pe) {
  HostContext* c = ctx(ctx_idx);
  if (!c) return -1;
  const Team* t = teams->get(c->team_slot);
  if (!t) return -1;
  return t->pe_in_world(pe);
}

int bshmem_runtime::group_of_team(int slot, CollGroup* g) {
  const Team* t = teams->get(slot);
  if (!t || t->my_pe < 0) return BSHMEM_ERR_INVALID;
  g->set = t->wrt_world;
  g->my_idx = t->my_pe;
  g->slot = slot;
  g->psync_off = 0;
  return BSHMEM_OK;
}

int bshmem_runtime::group_of_active_set(int start, int log_stride, int size, const long* psync, CollGroup* g) {
  if (start < 0 || log_stride < 0 || log_stride > 30 || size < 1) return BSHMEM_ERR_INVALID;
  TeamInfo s{start, 1 << log_stride, size};
  if (s.pe_at(size - 1) >= backend->n_pes()) return BSHMEM_ERR_INVALID;
  int idx = s.index_of(backend->my_pe());
  if (idx < 0) return BSHMEM_ERR_INVALID;
  uint64_t off = 0;
  if (!to_offset(psync, sizeof(long) * 2, &off)) return BSHMEM_ERR_RANGE;
  g->set = s;
  g->my_idx = idx;
  g->slot = -1;
  g->psync_off = off;
  return BSHMEM_OK;
}

bshmem_runtime* bshmem::make_runtime(std::unique_ptr<Backend> be, const bshmem_config_t* cfg) {
  bshmem_config_t c;
  if (cfg) c = *cfg; else bshmem_config_default(&c);
  if (c.max_teams < 1 || c.max_teams > BSHMEM_MAX_TEAMS) c.max_teams = BSHMEM_MAX_TEAMS;
  if (c.max_ctxs < 1 || c.max_ctxs > BSHMEM_MAX_CTXS) c.max_ctxs = BSHMEM_MAX_CTXS;
  if (c.timeout_us == 0) c.timeout_us = 30ull * 1000 * 1000;
  return new bshmem_runtime(std::move(be), c);
}

#define CHECK_H(h) do { if (!valid_handle(h)) return BSHMEM_ERR_STATE; } while (0)
#define STAT(h, c, idx, ...) do { (h)->global_stats.inc(idx, ##__VA_ARGS__); if (c) (c)->stats.inc(idx, ##__VA_ARGS__); } while (0)

extern "C" {

void bshmem_config_default(bshmem_config_t* cfg) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->heap_bytes = 1ull << 30;
  cfg->timeout_us = 30ull * 1000 * 1000;
  cfg->max_teams = BSHMEM_MAX_TEAMS;
  cfg->max_ctxs = BSHMEM_MAX_CTXS;
  cfg->debug = 0;
  cfg->profile = 1;
  cfg->requested_thread_level = BSHMEM_THREAD_MULTIPLE;
}

const char* bshmem_status_string(int s) {
  switch (s) {
    case BSHMEM_OK: return "ok";
    case BSHMEM_ERR_INVALID: return "invalid argument";
    case BSHMEM_ERR_NOMEM: return "symmetric heap exhausted";
    case BSHMEM_ERR_TIMEOUT: return "wait timed out";
    case BSHMEM_ERR_RANGE: return "address outside the symmetric heap";
    case BSHMEM_ERR_STATE: return "runtime not initialised";
    case BSHMEM_ERR_LIMIT: return "out of team or context slots";
    case BSHMEM_ERR_CUDA: return "CUDA error";
    case BSHMEM_ERR_UNSUPPORTED: return "unsupported";
    case BSHMEM_ERR_ABORTED: return "job aborted by global_exit";
    case BSHMEM_ERR_PEER_DEAD: return "peer marked failed";
    default: return "unknown";
  }
}

int bshmem_set_timeout_us(bshmem_handle_t h, uint64_t timeout_us) {
  CHECK_H(h);
  if (timeout_us == 0) return BSHMEM_ERR_INVALID;
  h->cfg.timeout_us = timeout_us;
  h->backend->set_timeout_us(timeout_us);
  return BSHMEM_OK;
}
uint64_t bshmem_get_timeout_us(bshmem_handle_t h) { return valid_handle(h) ? h->cfg.timeout_us : 0; }

void bshmem_set_current(bshmem_handle_t h) { tls_current = h; }
bshmem_handle_t bshmem_get_current(void) { return tls_current; }

int bshmem_finalize(bshmem_handle_t h) {
  CHECK_H(h);
  // Leftover contexts and teams are destroyed here, as in the reference.
  for (size_t i = 1; i < h->ctxs.size(); ++i)
    if (h->ctxs[i] && h->ctxs[i]->live) bshmem_ctx_destroy(h, (int)i);
  for (int s = 1; s < h->teams->max_teams(); ++s)
    if (h->teams->get(s)) h->backend->reset_slot(s);
  h->teams->destroy_all();
  h->backend->quiet();
  h->finalized = true;
  h->backend.reset();
  if (tls_current == h) tls_current = nullptr;
  delete h;
  return BSHMEM_OK;
}

int bshmem_query_thread(bshmem_handle_t h, int* provided) {
  CHECK_H(h);
  if (provided) *provided = BSHMEM_THREAD_MULTIPLE;   // host side is always MULTIPLE
  return BSHMEM_OK;
}

int bshmem_my_pe(bshmem_handle_t h) { return valid_handle(h) ? h->backend->my_pe() : -1; }
int bshmem_n_pes(bshmem_handle_t h) { return valid_handle(h) ? h->backend->n_pes() : -1; }

int bshmem_global_exit(bshmem_handle_t h, int status) {
  CHECK_H(h);
  return h->backend->global_exit(status);
}

const char* bshmem_last_error(bshmem_handle_t h) {
  if (!h) return "no handle";
  static thread_local std::string buf;
  {
    std::lock_guard<std::mutex> g(h->mu);
    buf = h->last_error;
  }
  if (buf.empty() && h->backend) buf = h->backend->last_error();
  return buf.c_str();
}

int bshmem_get_error_record(bshmem_handle_t h, bshmem_error_record_t* out, int clear) {
  CHECK_H(h);
  if (!out) return BSHMEM_ERR_INVALID;
  *out = h->backend->last_record(clear != 0);
  return BSHMEM_OK;
}

/* ---- memory ---------------------------------------------------------------- */
void* bshmem_malloc_local(bshmem_handle_t h, size_t size, size_t alignment) {
  if (!valid_handle(h)) return nullptr;
  uint64_t off = h->heap->alloc_aligned(size, alignment ? alignment : BSHMEM_ALIGNMENT);
  if (off == kNoOffset) {
    if (size) h->fail(BSHMEM_ERR_NOMEM, "symmetric heap exhausted");
    return nullptr;
  }
  STAT(h, (HostContext*)nullptr, ST_MALLOC);
  return h->backend->local_base() + off;
}

int bshmem_free_local(bshmem_handle_t h, void* ptr) {
  CHECK_H(h);
  if (!ptr) return BSHMEM_OK;
  uint64_t off;
  if (!h->to_offset(ptr, 0, &off)) return h->fail(BSHMEM_ERR_RANGE, "free: not a symmetric address");
  if (!h->heap->free(off)) return h->fail(BSHMEM_ERR_INVALID, "free: not the start of a live block");
  STAT(h, (HostContext*)nullptr, ST_FREE);
  return BSHMEM_OK;
}

void* bshmem_align(bshmem_handle_t h, size_t alignment, size_t size) {
  if (!valid_handle(h)) return nullptr;
  void* p = bshmem_malloc_local(h, size, alignment);
  // Collective: every PE leaves together so the block is usable remotely.
  if (bshmem_barrier_all(h) != BSHMEM_OK) { /* keep the block; the error is recorded */ }
  return p;
}

void* bshmem_malloc(bshmem_handle_t h, size_t size) { return bshmem_align(h, BSHMEM_ALIGNMENT, size); }

void* bshmem_calloc(bshmem_handle_t h, size_t count, size_t size) {
  if (!valid_handle(h)) return nullptr;
  if (count && size > SIZE_MAX / count) return nullptr;
  void* p = bshmem_malloc_local(h, count * size, BSHMEM_ALIGNMENT);
  if (p) {
    uint64_t off = 0;
    h->to_offset(p, 0, &off);
    h->backend->zero_local(off, count * size);
  }
  bshmem_barrier_all(h);
  return p;
}

int bshmem_free(bshmem_handle_t h, void* ptr) {
  CHECK_H(h);
  int rc = bshmem_barrier_all(h);   // nobody may still be targeting the block
  int rc2 = bshmem_free_local(h, ptr);
  return rc != BSHMEM_OK ? rc : rc2;
}

void* bshmem_ptr(bshmem_handle_t h, const void* dest, int pe) {
  if (!valid_handle(h)) return nullptr;
  uint64_t off;
  if (pe < 0 || pe >= h->backend->n_pes() || !h->to_offset(dest, 0, &off)) return nullptr;
  char* b = h->backend->peer_base(pe);
  return b ? b + off : nullptr;
}

void* bshmem_heap_base(bshmem_handle_t h) { return valid_handle(h) ? h->backend->local_base() : nullptr; }
uint64_t bshmem_heap_bytes(bshmem_handle_t h) { return valid_handle(h) ? h->backend->heap_bytes() : 0; }

int bshmem_heap_usage(bshmem_handle_t h, uint64_t out[9]) {
  CHECK_H(h);
  HeapUsage u = h->heap->usage();
  out[0] = u.heap_bytes; out[1] = u.reserved_bytes; out[2] = u.allocated_bytes; out[3] = u.requested_bytes;
  out[4] = u.live_blocks; out[5] = u.largest_free; out[6] = u.n_allocs; out[7] = u.n_frees; out[8] = u.n_failed;
  return BSHMEM_OK;
}

int bshmem_addr_accessible(bshmem_handle_t h, const void* addr, int pe) {
  if (!valid_handle(h)) return 0;
  uint64_t off;
  return (pe >= 0 && pe < h->backend->n_pes() && h->to_offset(addr, 0, &off)) ? 1 : 0;
}

/* ---- contexts -------------------------------------------------------------- */
namespace {
// The backend operations issued inside this scope belong to host context `c`.
struct CtxScope {
  Backend* be;
  CtxScope(bshmem_handle_t h, int c) : be(h->backend.get()) { be->ctx_select(c); }
  ~CtxScope() { be->ctx_select(0); }
};
}  // namespace

int bshmem_team_create_ctx(bshmem_handle_t h, bshmem_team_t team, long options, bshmem_ctx_t* out) {
  CHECK_H(h);
  if (!out) return BSHMEM_ERR_INVALID;
  *out = BSHMEM_CTX_INVALID;
  const Team* t = h->teams->get(team);
  if (!t || t->my_pe < 0) return h->fail(BSHMEM_ERR_INVALID, "ctx_create: invalid team");
  std::lock_guard<std::mutex> g(h->mu);
  for (size_t i = 1; i < h->ctxs.size(); ++i) {
    if (!h->ctxs[i] || !h->ctxs[i]->live) {
      int rc = h->backend->ctx_open((int)i, options);
      if (rc != BSHMEM_OK) return h->fail(rc, "ctx_create: the backend could not open the context");
      h->ctxs[i].reset(new HostContext());
      h->ctxs[i]->live = true;
      h->ctxs[i]->options = options;
      h->ctxs[i]->owner = std::this_thread::get_id();
      h->ctxs[i]->team_slot = team;
      h->ctxs[i]->stats.enable(h->cfg.profile != 0);
      *out = (bshmem_ctx_t)i;
      h->global_stats.inc(ST_CTX_CREATE);
      return BSHMEM_OK;
    }
  }
  return BSHMEM_ERR_LIMIT;
}

int bshmem_ctx_create(bshmem_handle_t h, long options, bshmem_ctx_t* out) {
  return bshmem_team_create_ctx(h, BSHMEM_TEAM_WORLD, options, out);
}

int bshmem_ctx_destroy(bshmem_handle_t h, bshmem_ctx_t c) {
  CHECK_H(h);
  if (c == BSHMEM_CTX_DEFAULT) return BSHMEM_OK;   // the default context lives until finalize
  HostContext* x = h->ctx(c);
  if (!x) return BSHMEM_ERR_INVALID;
  {
    CtxScope sel(h, c);
    h->backend->quiet();   // destroying a context completes its operations
  }
  h->backend->ctx_close(c);
  std::lock_guard<std::mutex> g(h->mu);
  x->live = false;
  h->global_stats.inc(ST_CTX_DESTROY);
  return BSHMEM_OK;
}

/* ---- teams ----------------------------------------------------------------- */
int bshmem_team_split_strided(bshmem_handle_t h, bshmem_team_t parent, int start, int stride, int size,
                              bshmem_team_t* new_team) {
  CHECK_H(h);
  if (!new_team) return BSHMEM_ERR_INVALID;
  *new_team = BSHMEM_TEAM_INVALID;
  if (parent == BSHMEM_TEAM_INVALID) return BSHMEM_OK;
  Team planned;
  bool member = false;
  int rc = h->teams->plan_split(parent, start, stride, size, &planned, &member);
  if (rc != BSHMEM_OK) return h->fail(rc, "team_split_strided: bad start/stride/size");
  // Collective over the parent: everyone publishes its free-slot mask; the new
  // team's members intersect theirs and take the lowest common slot.
  CollGroup pg;
  rc = h->group_of_team(parent, &pg);
  if (rc != BSHMEM_OK) return h->fail(rc, "team_split_strided: caller is not in the parent team");
  uint64_t masks[BSHMEM_MAX_PES];
  rc = h->backend->exchange_u64(pg, h->teams->free_mask(), masks);
  if (rc != BSHMEM_OK) return h->fail(rc, "team_split_strided: slot agreement failed");
  h->global_stats.inc(ST_TEAM_SPLIT);
  if (!member) return BSHMEM_OK;
  uint64_t m = ~0ull;
  for (int i = 0; i < size; ++i) m &= masks[planned.wrt_parent.pe_at(i)];
  int slot = TeamTracker::pick_slot(m);
  if (slot < 0) return h->fail(BSHMEM_ERR_LIMIT, "team_split_strided: no common free team slot");
  rc = h->teams->commit(planned, slot);
  if (rc != BSHMEM_OK) return rc;
  *new_team = slot;
  return BSHMEM_OK;
}

int bshmem_team_destroy(bshmem_handle_t h, bshmem_team_t team) {
  CHECK_H(h);
  if (team <= 0) return BSHMEM_OK;
  h->global_stats.inc(ST_TEAM_DESTROY);
  if (!h->teams->get(team)) return BSHMEM_OK;
  h->backend->reset_slot(team);
  return h->teams->destroy(team);
}

int bshmem_team_n_pes(bshmem_handle_t h, bshmem_team_t team) {
  if (!valid_handle(h)) return -1;
  const Team* t = h->teams->get(team);
  return t ? t->num_pes : -1;
}

int bshmem_team_my_pe(bshmem_handle_t h, bshmem_team_t team) {
  if (!valid_handle(h)) return -1;
  const Team* t = h->teams->get(team);
  return t ? t->my_pe : -1;
}

int bshmem_team_translate_pe(bshmem_handle_t h, bshmem_team_t src, int src_pe, bshmem_team_t dst) {
  if (!valid_handle(h)) return -1;
  const Team* a = h->teams->get(src);
  const Team* b = h->teams->get(dst);
  if (!a || !b) return -1;
  return team_translate_pe(*a, src_pe, *b);
}

/* ---- RMA ------------------------------------------------------------------- */

static int do_put(bshmem_handle_t h, int c, void* dest, const void* src, size_t n, int pe, bool nbi) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return h->fail(BSHMEM_ERR_INVALID, "put: invalid context");
  if (n == 0) return BSHMEM_OK;
  int wpe = h->resolve_pe(c, pe);
  uint64_t off;
  if (wpe < 0) return h->fail(BSHMEM_ERR_INVALID, "put: PE out of range");
  if (!src) return h->fail(BSHMEM_ERR_INVALID, "put: null source");
  if (!h->to_offset(dest, n, &off)) return h->fail(BSHMEM_ERR_RANGE, "put: dest is not symmetric");
  STAT(h, x, nbi ? ST_PUT_NBI : ST_PUT);
  STAT(h, x, ST_BYTES_PUT, n);
  CtxScope sel(h, c);
  return h->backend->put(wpe, off, src, n, nbi);
}

static int do_get(bshmem_handle_t h, int c, void* dest, const void* src, size_t n, int pe, bool nbi) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return h->fail(BSHMEM_ERR_INVALID, "get: invalid context");
  if (n == 0) return BSHMEM_OK;
  int wpe = h->resolve_pe(c, pe);
  uint64_t off;
  if (wpe < 0) return h->fail(BSHMEM_ERR_INVALID, "get: PE out of range");
  if (!dest) return h->fail(BSHMEM_ERR_INVALID, "get: null dest");
  if (!h->to_offset(src, n, &off)) return h->fail(BSHMEM_ERR_RANGE, "get: source is not symmetric");
  STAT(h, x, nbi ? ST_GET_NBI : ST_GET);
  STAT(h, x, ST_BYTES_GET, n);
  CtxScope sel(h, c);
  return h->backend->get(wpe, dest, off, n, nbi);
}

int bshmem_ctx_putmem(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, int pe) { return do_put(h, c, d, s, n, pe, false); }
int bshmem_ctx_putmem_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, int pe) { return do_put(h, c, d, s, n, pe, true); }
int bshmem_ctx_getmem(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, int pe) { return do_get(h, c, d, s, n, pe, false); }
int bshmem_ctx_getmem_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, int pe) { return do_get(h, c, d, s, n, pe, true); }

static int do_put_signal(bshmem_handle_t h, int c, void* dest, const void* src, size_t n, uint64_t* sig,
                         uint64_t val, int sig_op, int pe, bool nbi) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return h->fail(BSHMEM_ERR_INVALID, "put_signal: invalid context");
  int wpe = h->resolve_pe(c, pe);
  if (wpe < 0) return h->fail(BSHMEM_ERR_INVALID, "put_signal: PE out of range");
  if (sig_op != BSHMEM_SIGNAL_SET && sig_op != BSHMEM_SIGNAL_ADD) return h->fail(BSHMEM_ERR_INVALID, "put_signal: bad signal op");
  uint64_t off = 0, soff;
  if (n && !h->to_offset(dest, n, &off)) return h->fail(BSHMEM_ERR_RANGE, "put_signal: dest is not symmetric");
  if (!h->to_offset(sig, 8, &soff) || (soff & 7)) return h->fail(BSHMEM_ERR_RANGE, "put_signal: signal word is not symmetric / aligned");
  STAT(h, x, ST_PUT_SIGNAL);
  STAT(h, x, ST_BYTES_PUT, n);
  CtxScope sel(h, c);
  return h->backend->put_signal(wpe, off, src, n, soff, val, sig_op, nbi);
}

int bshmem_ctx_putmem_signal(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, uint64_t* sig,
                             uint64_t v, int op, int pe) { return do_put_signal(h, c, d, s, n, sig, v, op, pe, false); }
int bshmem_ctx_putmem_signal_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* d, const void* s, size_t n, uint64_t* sig,
                                 uint64_t v, int op, int pe) { return do_put_signal(h, c, d, s, n, sig, v, op, pe, true); }

uint64_t bshmem_signal_fetch(bshmem_handle_t h, const uint64_t* sig) {
  if (!valid_handle(h)) return 0;
  uint64_t off, out = 0;
  if (!h->to_offset(sig, 8, &off)) return 0;
  h->backend->amo(h->backend->my_pe(), off, BSHMEM_UINT64, BSHMEM_AMO_FETCH, 0, 0, &out);
  return out;
}

int bshmem_ctx_amo(bshmem_handle_t h, bshmem_ctx_t c, int dtype, int op, void* dest, uint64_t value, uint64_t cond,
                   int pe, uint64_t* fetched) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return h->fail(BSHMEM_ERR_INVALID, "amo: invalid context");
  if (op < 0 || op >= BSHMEM_AMO_COUNT) return h->fail(BSHMEM_ERR_INVALID, "amo: bad op");
  size_t sz = bshmem_dtype_size(dtype);
  if (sz != 4 && sz != 8) return h->fail(BSHMEM_ERR_UNSUPPORTED, "amo: only 4- and 8-byte types");
  int wpe = h->resolve_pe(c, pe);
  if (wpe < 0) return h->fail(BSHMEM_ERR_INVALID, "amo: PE out of range");
  uint64_t off;
  if (!h->to_offset(dest, sz, &off) || (off & (sz - 1))) return h->fail(BSHMEM_ERR_RANGE, "amo: dest is not symmetric / aligned");
  STAT(h, x, kAmoStat[op]);
  uint64_t tmp = 0;
  CtxScope sel(h, c);
  int rc = h->backend->amo(wpe, off, dtype, op, value, cond, &tmp);
  if (fetched) *fetched = tmp;
  return rc;
}

/* ---- ordering / sync --------------------------------------------------------- */
int bshmem_ctx_fence(bshmem_handle_t h, bshmem_ctx_t c) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return BSHMEM_ERR_INVALID;
  STAT(h, x, ST_FENCE);
  CtxScope sel(h, c);
  return h->backend->fence();
}

int bshmem_ctx_quiet(bshmem_handle_t h, bshmem_ctx_t c) {
  CHECK_H(h);
  HostContext* x = h->ctx(c);
  if (!x) return BSHMEM_ERR_INVALID;
  STAT(h, x, ST_QUIET);
  CtxScope sel(h, c);
  return h->backend->quiet();
}

int bshmem_wait_until(bshmem_handle_t h, int dtype, void* ivar, int cmp, uint64_t value) {
  CHECK_H(h);
  size_t sz = bshmem_dtype_size(dtype);
  uint64_t off;
  if (cmp < BSHMEM_CMP_EQ || cmp > BSHMEM_CMP_LE) return h->fail(BSHMEM_ERR_INVALID, "wait_until: bad comparator");
  if (!sz || !h->to_offset(ivar, sz, &off) || (off & (sz - 1))) return h->fail(BSHMEM_ERR_RANGE, "wait_until: ivar is not symmetric / aligned");
  STAT(h, h->ctx(0), ST_WAIT_UNTIL);
  int rc = h->backend->wait_until(off, dtype, cmp, value, h->cfg.timeout_us);
  if (rc == BSHMEM_ERR_TIMEOUT) { STAT(h, h->ctx(0), ST_TIMEOUTS); h->fail(rc, "wait_until timed out"); }
  return rc;
}

int bshmem_test(bshmem_handle_t h, int dtype, void* ivar, int cmp, uint64_t value, int* result) {
  CHECK_H(h);
  size_t sz = bshmem_dtype_size(dtype);
  uint64_t off;
  if (!result || cmp < BSHMEM_CMP_EQ || cmp > BSHMEM_CMP_LE) return BSHMEM_ERR_INVALID;
  if (!sz || !h->to_offset(ivar, sz, &off) || (off & (sz - 1))) return h->fail(BSHMEM_ERR_RANGE, "test: ivar is not symmetric / aligned");
  STAT(h, h->ctx(0), ST_TEST);
  return h->backend->test(off, dtype, cmp, value, result);
}

/* ---- collectives -------------------------------------------------------------- */
static int note_timeout(bshmem_handle_t h, int rc, const char* what) {
  if (rc == BSHMEM_ERR_TIMEOUT) { h->global_stats.inc(ST_TIMEOUTS); h->fail(rc, std::string(what) + " timed out"); }
  else if (rc != BSHMEM_OK) h->fail(rc, std::string(what) + ": " + bshmem_status_string(rc));
  return rc;
}

int bshmem_team_sync(bshmem_handle_t h, bshmem_team_t team) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "team_sync: invalid team");
  h->global_stats.inc(team == 0 ? ST_SYNC_ALL : ST_TEAM_SYNC);
  return note_timeout(h, h->backend->sync(g), "team_sync");
}

int bshmem_team_barrier(bshmem_handle_t h, bshmem_team_t team) {
  CHECK_H(h);
  int rc = h->backend->quiet();   // barrier = quiet + sync
  if (rc != BSHMEM_OK) return rc;
  return bshmem_team_sync(h, team);
}

int bshmem_sync_all(bshmem_handle_t h) { return bshmem_team_sync(h, BSHMEM_TEAM_WORLD); }

int bshmem_barrier_all(bshmem_handle_t h) {
  CHECK_H(h);
  h->global_stats.inc(ST_BARRIER_ALL);
  return bshmem_team_barrier(h, BSHMEM_TEAM_WORLD);
}

static int coll_offsets(bshmem_handle_t h, void* dest, size_t dbytes, const void* src, size_t sbytes,
                        uint64_t* doff, uint64_t* soff, const char* what) {
  if (!h->to_offset(dest, dbytes, doff)) return h->fail(BSHMEM_ERR_RANGE, std::string(what) + ": dest is not symmetric");
  if (!h->to_offset(src, sbytes, soff)) return h->fail(BSHMEM_ERR_RANGE, std::string(what) + ": source is not symmetric");
  return BSHMEM_OK;
}

static int bcast_impl(bshmem_handle_t h, const CollGroup& g, void* dest, const void* src, size_t nbytes, int root) {
  if (root < 0 || root >= g.size()) return h->fail(BSHMEM_ERR_INVALID, "broadcast: root outside the set");
  uint64_t doff, soff;
  int rc = coll_offsets(h, dest, nbytes, src, nbytes, &doff, &soff, "broadcast");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_BROADCAST);
  return note_timeout(h, h->backend->broadcast(g, doff, soff, nbytes, root), "broadcast");
}

int bshmem_team_broadcast(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src, size_t nbytes, int root) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "broadcast: invalid team");
  return bcast_impl(h, g, dest, src, nbytes, root);
}

static int reduce_impl(bshmem_handle_t h, const CollGroup& g, int dtype, int op, void* dest, const void* src, size_t nelems) {
  size_t sz = bshmem_dtype_size(dtype);
  if (!sz || op < BSHMEM_SUM || op > BSHMEM_XOR) return h->fail(BSHMEM_ERR_INVALID, "to_all: bad dtype/op");
  bool is_float = dtype >= BSHMEM_FLOAT;
  if (is_float && op >= BSHMEM_AND) return h->fail(BSHMEM_ERR_INVALID, "to_all: bitwise op on a floating type");
  uint64_t doff, soff;
  int rc = coll_offsets(h, dest, nelems * sz, src, nelems * sz, &doff, &soff, "to_all");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_TO_ALL);
  return note_timeout(h, h->backend->reduce(g, dtype, op, doff, soff, nelems), "to_all");
}

int bshmem_team_reduce(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest, const void* src, size_t nelems) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "to_all: invalid team");
  return reduce_impl(h, g, dtype, op, dest, src, nelems);
}

int bshmem_team_reduce_root(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest, const void* src, size_t nelems,
                            int root) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "reduce: invalid team");
  if (root < 0 || root >= g.size()) return h->fail(BSHMEM_ERR_INVALID, "reduce: root is not a member of the team");
  size_t sz = bshmem_dtype_size(dtype);
  if (!sz || op < BSHMEM_SUM || op > BSHMEM_XOR || (dtype >= BSHMEM_FLOAT && op >= BSHMEM_AND))
    return h->fail(BSHMEM_ERR_INVALID, "reduce: bad dtype/op");
  uint64_t doff, soff;
  rc = coll_offsets(h, dest, nelems * sz, src, nelems * sz, &doff, &soff, "reduce");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_TO_ALL);
  return note_timeout(h, h->backend->reduce_root(g, dtype, op, doff, soff, nelems, root), "reduce");
}

int bshmem_team_reduce_scatter(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest, const void* src,
                               size_t nelems_per_pe) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "reduce_scatter: invalid team");
  size_t sz = bshmem_dtype_size(dtype);
  if (!sz || op < BSHMEM_SUM || op > BSHMEM_XOR || (dtype >= BSHMEM_FLOAT && op >= BSHMEM_AND))
    return h->fail(BSHMEM_ERR_INVALID, "reduce_scatter: bad dtype/op");
  uint64_t doff, soff;
  rc = coll_offsets(h, dest, nelems_per_pe * sz, src, nelems_per_pe * sz * g.size(), &doff, &soff, "reduce_scatter");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_REDUCE_SCATTER);
  return note_timeout(h, h->backend->reduce_scatter(g, dtype, op, doff, soff, nelems_per_pe), "reduce_scatter");
}

int bshmem_team_fcollect(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src, size_t nbytes) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "fcollect: invalid team");
  uint64_t doff, soff;
  rc = coll_offsets(h, dest, nbytes * g.size(), src, nbytes, &doff, &soff, "fcollect");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_FCOLLECT);
  return note_timeout(h, h->backend->fcollect(g, doff, soff, nbytes), "fcollect");
}

int bshmem_team_alltoall(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src, size_t nbytes) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_team(team, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "alltoall: invalid team");
  uint64_t doff, soff;
  rc = coll_offsets(h, dest, nbytes * g.size(), src, nbytes * g.size(), &doff, &soff, "alltoall");
  if (rc != BSHMEM_OK) return rc;
  h->global_stats.inc(ST_ALLTOALL);
  return note_timeout(h, h->backend->alltoall(g, doff, soff, nbytes), "alltoall");
}

/* ---- active-set forms --------------------------------------------------------- */
int bshmem_sync(bshmem_handle_t h, int pe_start, int log_stride, int pe_size, long* psync) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_active_set(pe_start, log_stride, pe_size, psync, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "sync: bad active set or pSync");
  return note_timeout(h, h->backend->sync(g), "sync");
}

int bshmem_barrier(bshmem_handle_t h, int pe_start, int log_stride, int pe_size, long* psync) {
  CHECK_H(h);
  int rc = h->backend->quiet();
  if (rc != BSHMEM_OK) return rc;
  return bshmem_sync(h, pe_start, log_stride, pe_size, psync);
}

int bshmem_broadcast(bshmem_handle_t h, void* dest, const void* src, size_t nbytes, int root, int pe_start,
                     int log_stride, int pe_size, long* psync) {
  CHECK_H(h);
  CollGroup g;
  int rc = h->group_of_active_set(pe_start, log_stride, pe_size, psync, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "broadcast: bad active set or pSync");
  return bcast_impl(h, g, dest, src, nbytes, root);
}

int bshmem_to_all(bshmem_handle_t h, int dtype, int op, void* dest, const void* src, size_t nelems, int pe_start,
                  int log_stride, int pe_size, void* pwrk, long* psync) {
  CHECK_H(h);
  (void)pwrk;   // reductions read the peers' sources in place; no work array is needed
  CollGroup g;
  int rc = h->group_of_active_set(pe_start, log_stride, pe_size, psync, &g);
  if (rc != BSHMEM_OK) return h->fail(rc, "to_all: bad active set or pSync");
  return reduce_impl(h, g, dtype, op, dest, src, nelems);
}

/* ---- statistics ----------------------------------------------------------------- */
int bshmem_stats_count(void) { return ST_COUNT; }
const char* bshmem_stats_name(int idx) { return host_stat_name(idx); }

int bshmem_get_stats(bshmem_handle_t h, uint64_t* out, int n) {
  CHECK_H(h);
  for (int i = 0; i < n && i < ST_COUNT; ++i) out[i] = h->global_stats.get(i);
  return BSHMEM_OK;
}

int bshmem_reset_stats(bshmem_handle_t h) {
  CHECK_H(h);
  h->global_stats.reset();
  for (auto& c : h->ctxs) if (c) c->stats.reset();
  return BSHMEM_OK;
}

int bshmem_dump_stats(bshmem_handle_t h) {
  CHECK_H(h);
  printf("[bshmem pe %d/%d, backend %s] host API counters\n", h->backend->my_pe(), h->backend->n_pes(), h->backend->name());
  for (int i = 0; i < ST_COUNT; ++i) {
    uint64_t v = h->global_stats.get(i);
    if (v) printf("  %-18s %llu\n", host_stat_name(i), (unsigned long long)v);
  }
  fflush(stdout);
  return BSHMEM_OK;
}

}  // extern "C"
