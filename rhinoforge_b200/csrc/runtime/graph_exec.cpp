// Native graph runtime: a signature-indexed cache of captured CUDA graphs.
//
// A capture scope is `begin(signature) ... launches ... end()`:
//   * first time (BUILD): the stream is put into capture, the launches between
//     begin and end are recorded, end() instantiates the graph and launches it
//     once, so a BUILD call also produces its result;
//   * afterwards (REPLAY): begin() switches this thread's launchers to "skip"
//     mode -- the same host code may walk the same launch sequence, nothing is
//     enqueued -- and end() launches the stored executable graph.
// Values that change between replays (positions, page tables, token ids) live in
// device buffers at stable addresses, so a replay needs no node updates.
//
// B200 counterpart of the reference's RpuKernelGraph / RpuGraphCache
// (src/graph/graph_runtime.h:1126-1133 state machine, :1050-1120 stats,
// src/graph/graph_infra.h:40-130 signature + hash, :558-634 cache + snapshot).
#include <stdint.h>
#include <string.h>

#include <list>
#include <memory>
#include <mutex>
#include <sstream>
#include <unordered_map>
#include <vector>

#include "../common/host_util.h"
#include "../rf_api.h"
#include "handle_registry.h"

namespace rf {

enum GraphState : int32_t { kPassthrough = 0, kRecording = 1, kBuilt = 2, kReplaying = 3 };

struct Signature {
  std::vector<int64_t> words;  // [op_id, flags, branch, segment, n_shapes, shapes.., n_dyn, dyn.., n_dt, dt..]
  bool operator==(const Signature& o) const { return words == o.words; }
  uint64_t hash() const {
    uint64_t h = 0xCBF29CE484222325ull;
    for (int64_t w : words) {
      for (int b = 0; b < 8; ++b) {
        h ^= (uint64_t)(w >> (8 * b)) & 0xffu;
        h *= 0x100000001B3ull;
      }
    }
    return h;
  }
  int64_t op_id() const { return words.empty() ? 0 : words[0]; }
  std::string str() const {
    std::ostringstream os;
    os << "sig[";
    for (size_t i = 0; i < words.size(); ++i) os << (i ? "," : "") << words[i];
    os << "]";
    return os.str();
  }
};
struct SigHash {
  size_t operator()(const Signature& s) const { return (size_t)s.hash(); }
};

struct GraphEntry {
  Signature sig;
  GraphState state = kPassthrough;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t build_count = 0, replay_count = 0, recapture_count = 0, node_count = 0, launch_count_at_build = 0;
  std::string non_replayable_reason;
  ~GraphEntry() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
  }
};

struct GraphCacheImpl {
  int max_entries = 32;
  std::mutex mu;
  std::list<std::shared_ptr<GraphEntry>> lru;  // front = most recent
  std::unordered_map<Signature, std::list<std::shared_ptr<GraphEntry>>::iterator, SigHash> index;
  std::shared_ptr<GraphEntry> active;  // entry between begin and end on this cache
  cudaStream_t active_stream = nullptr;
  uint64_t launches_before = 0;
  uint64_t evictions = 0;
};

static HandleRegistry<GraphCacheImpl>& caches() {
  static HandleRegistry<GraphCacheImpl> r;
  return r;
}

static thread_local int g_replay_depth = 0;
bool replay_mode() { return g_replay_depth > 0; }

static Signature make_sig(const int64_t* words, int n) {
  Signature s;
  s.words.assign(words, words + n);
  return s;
}

}  // namespace rf

using namespace rf;

extern "C" uint64_t rf_launch_count(void);

extern "C" int64_t rf_graphcache_create(int32_t max_entries) {
  auto c = std::make_unique<GraphCacheImpl>();
  c->max_entries = max_entries > 0 ? max_entries : 32;
  return caches().insert(std::move(c));
}

extern "C" int rf_graphcache_destroy(int64_t h) {
  return caches().erase(h) ? RF_OK : fail(RF_ERR_BAD_ARG, "unknown graph cache %lld", (long long)h);
}

#define RF_GET_CACHE(h)                                                               \
  std::shared_ptr<GraphCacheImpl> cp = caches().get(h);                               \
  if (!cp) return fail(RF_ERR_BAD_ARG, "unknown graph cache %lld", (long long)(h));   \
  GraphCacheImpl& c = *cp;

// Returns the state the scope runs in through *state_out: kRecording (BUILD) or kReplaying.
// allow_build == 0 (frozen cache): a miss or a non-BUILT entry is an error.
extern "C" int rf_graph_begin(int64_t h, const int64_t* words, int32_t n, rf_stream_t stream_, int32_t allow_build,
                              int32_t* state_out) {
  RF_GET_CACHE(h);
  RF_REQUIRE(words && n >= 4, "graph signature needs at least 4 words");
  std::lock_guard<std::mutex> g(c.mu);
  RF_REQUIRE(!c.active, "graph scope already open on this cache (nested capture is not supported)");
  Signature sig = make_sig(words, n);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::shared_ptr<GraphEntry> e;
  auto it = c.index.find(sig);
  if (it != c.index.end()) {
    e = *it->second;
    c.lru.splice(c.lru.begin(), c.lru, it->second);
  } else {
    if (!allow_build) return fail(RF_ERR_STATE, "graph cache is frozen: miss for %s", sig.str().c_str());
    e = std::make_shared<GraphEntry>();
    e->sig = sig;
    while ((int)c.lru.size() >= c.max_entries) {
      c.index.erase(c.lru.back()->sig);
      c.lru.pop_back();
      ++c.evictions;
    }
    c.lru.push_front(e);
    c.index[sig] = c.lru.begin();
  }
  if (e->state == kBuilt) {
    e->state = kReplaying;
    ++g_replay_depth;
  } else {
    if (!allow_build) return fail(RF_ERR_STATE, "graph cache is frozen: entry %s is not built", sig.str().c_str());
    if (e->exec) { cudaGraphExecDestroy(e->exec); e->exec = nullptr; ++e->recapture_count; }
    if (e->graph) { cudaGraphDestroy(e->graph); e->graph = nullptr; }
    RF_CUDA_CHECK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    e->state = kRecording;
    c.launches_before = rf_launch_count();
  }
  c.active = e;
  c.active_stream = stream;
  if (state_out) *state_out = e->state;
  return RF_OK;
}

extern "C" int rf_graph_end(int64_t h) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  RF_REQUIRE(c.active != nullptr, "graph end without begin");
  std::shared_ptr<GraphEntry> e = c.active;
  cudaStream_t stream = c.active_stream;
  c.active.reset();
  if (e->state == kReplaying) {
    --g_replay_depth;
    e->state = kBuilt;
    RF_CUDA_CHECK(cudaGraphLaunch(e->exec, stream));
    ++e->replay_count;
    return RF_OK;
  }
  // RECORDING -> BUILT
  cudaGraph_t graph = nullptr;
  cudaError_t err = cudaStreamEndCapture(stream, &graph);
  if (err != cudaSuccess || graph == nullptr) {
    e->state = kPassthrough;
    e->non_replayable_reason = cudaGetErrorString(err);
    cudaGetLastError();
    return fail(RF_ERR_CUDA, "stream capture failed: %s", cudaGetErrorString(err));
  }
  e->graph = graph;
  size_t nodes = 0;
  cudaGraphGetNodes(graph, nullptr, &nodes);
  e->node_count = nodes;
  e->launch_count_at_build = rf_launch_count() - c.launches_before;
  err = cudaGraphInstantiate(&e->exec, graph, 0);
  if (err != cudaSuccess) {
    e->state = kPassthrough;
    e->non_replayable_reason = cudaGetErrorString(err);
    return fail(RF_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(err));
  }
  e->state = kBuilt;
  ++e->build_count;
  RF_CUDA_CHECK(cudaGraphLaunch(e->exec, stream));
  return RF_OK;
}

// Leave the scope after an exception: drop a half-recorded graph, keep a built one.
extern "C" int rf_graph_abort(int64_t h) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  if (!c.active) return RF_OK;
  std::shared_ptr<GraphEntry> e = c.active;
  c.active.reset();
  if (e->state == kReplaying) {
    --g_replay_depth;
    e->state = kBuilt;
    return RF_OK;
  }
  cudaGraph_t graph = nullptr;
  cudaStreamEndCapture(c.active_stream, &graph);
  if (graph) cudaGraphDestroy(graph);
  cudaGetLastError();
  e->state = kPassthrough;
  auto it = c.index.find(e->sig);
  if (it != c.index.end()) {
    c.lru.erase(it->second);
    c.index.erase(it);
  }
  return RF_OK;
}

// Replay a built entry directly (no scope, no host re-walk).
extern "C" int rf_graph_replay(int64_t h, const int64_t* words, int32_t n, rf_stream_t stream) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  auto it = c.index.find(make_sig(words, n));
  RF_REQUIRE(it != c.index.end() && (*it->second)->state == kBuilt, "graph replay: no built entry");
  GraphEntry& e = **it->second;
  RF_CUDA_CHECK(cudaGraphLaunch(e.exec, static_cast<cudaStream_t>(stream)));
  ++e.replay_count;
  return RF_OK;
}

extern "C" int32_t rf_graphcache_size(int64_t h) {
  auto cp = caches().get(h);
  if (!cp) return -1;
  std::lock_guard<std::mutex> g(cp->mu);
  return (int32_t)cp->lru.size();
}

extern "C" int32_t rf_graphcache_max_entries(int64_t h) {
  auto cp = caches().get(h);
  return cp ? cp->max_entries : -1;
}

// state of the entry for `words`, or -1 when absent
extern "C" int32_t rf_graphcache_lookup(int64_t h, const int64_t* words, int32_t n) {
  auto cp = caches().get(h);
  if (!cp) return -1;
  std::lock_guard<std::mutex> g(cp->mu);
  auto it = cp->index.find(make_sig(words, n));
  return it == cp->index.end() ? -1 : (int32_t)(*it->second)->state;
}

extern "C" int rf_graphcache_evict(int64_t h, const int64_t* words, int32_t n) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  auto it = c.index.find(make_sig(words, n));
  if (it == c.index.end()) return RF_OK;
  RF_REQUIRE(!(c.active && c.active == *it->second), "cannot evict the entry of an open scope");
  c.lru.erase(it->second);
  c.index.erase(it);
  return RF_OK;
}

extern "C" int rf_graphcache_clear(int64_t h) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  RF_REQUIRE(!c.active, "cannot clear a cache with an open scope");
  c.index.clear();
  c.lru.clear();
  return RF_OK;
}

// index and LRU list agree, every BUILT entry has an executable, size within bound
extern "C" int32_t rf_graphcache_invariant_ok(int64_t h) {
  auto cp = caches().get(h);
  if (!cp) return 0;
  std::lock_guard<std::mutex> g(cp->mu);
  if (cp->index.size() != cp->lru.size() || (int)cp->lru.size() > cp->max_entries) return 0;
  for (auto& e : cp->lru) {
    if (e->state == kBuilt && !e->exec) return 0;
    auto it = cp->index.find(e->sig);
    if (it == cp->index.end() || *it->second != e) return 0;
  }
  return 1;
}

// One line per entry: "op_id state builds replays recaptures nodes launches reason|words..."
extern "C" int rf_graphcache_snapshot(int64_t h, char* buf, int32_t cap) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  std::ostringstream os;
  for (auto& e : c.lru) {
    os << e->sig.op_id() << ' ' << (int)e->state << ' ' << e->build_count << ' ' << e->replay_count << ' '
       << e->recapture_count << ' ' << e->node_count << ' ' << e->launch_count_at_build << ' '
       << (e->non_replayable_reason.empty() ? "-" : "non-replayable") << '|';
    for (size_t i = 0; i < e->sig.words.size(); ++i) os << (i ? "," : "") << e->sig.words[i];
    os << '\n';
  }
  const std::string s = os.str();
  RF_REQUIRE(buf && cap > 0, "snapshot buffer");
  const size_t nbytes = std::min<size_t>(s.size(), (size_t)cap - 1);
  memcpy(buf, s.data(), nbytes);
  buf[nbytes] = 0;
  return (int)s.size() + 1 > cap ? RF_ERR_NO_MEMORY : RF_OK;
}

// Which signature word first differs from the closest cached entry (diagnostics for a miss).
extern "C" int rf_graphcache_explain_miss(int64_t h, const int64_t* words, int32_t n, char* buf, int32_t cap) {
  RF_GET_CACHE(h);
  std::lock_guard<std::mutex> g(c.mu);
  Signature sig = make_sig(words, n);
  std::string msg;
  if (c.index.count(sig)) {
    msg = "hit";
  } else {
    size_t best = 0;
    const GraphEntry* beste = nullptr;
    for (auto& e : c.lru) {
      size_t k = 0;
      while (k < e->sig.words.size() && k < sig.words.size() && e->sig.words[k] == sig.words[k]) ++k;
      if (!beste || k > best) { best = k; beste = e.get(); }
    }
    static const char* layer[] = {"GmId", "ScalarFlags", "BranchKey", "SegmentKey"};
    std::ostringstream os;
    if (!beste) os << "miss at GmId: cache is empty";
    else if (best < 4) os << "miss at " << layer[best] << ": word " << best << " differs";
    else os << "miss at ShapeBucket/DtypeLayout: word " << best << " differs from the closest entry " << beste->sig.str();
    msg = os.str();
  }
  RF_REQUIRE(buf && cap > 0, "explain buffer");
  strncpy(buf, msg.c_str(), cap - 1);
  buf[cap - 1] = 0;
  return RF_OK;
}

extern "C" int32_t rf_replay_mode(void) { return rf::replay_mode() ? 1 : 0; }
