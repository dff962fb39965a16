// Bounded retention of captured CUDA graphs, keyed by the shape of a verify window.
//
// Upstream replays one captured graph per (slot, parity, rows, geometry) of its speculative-verify windows and keeps
// them in a bounded cache (src/verifier_graph_cache.rs: Policy, Cache::{action, insert}; used by
// src/multi_decode.rs:470-537, where two to four requests share one <= 16-row expert call).  This is that policy
// behind the C ABI -- the same decisions (replay / run eagerly / capture), the same two caps (entries, graph nodes),
// least-recently-used eviction, bounded tracking of keys that were seen but not yet captured -- plus the capture
// itself: glmflash_graph_cache_run records the caller's enqueue function into a graph on first need and replays it
// afterwards.  The policy part needs no GPU.
#include <map>
#include <new>

#include "common.cuh"

struct glmflash_graph_cache {
    glmflash_graph_policy policy;
    struct Entry {
        cudaGraphExec_t exec;
        uint64_t nodes, used;
    };
    struct Seen {
        uint32_t count;
        uint64_t used;
    };
    std::map<uint64_t, Entry> entries;
    std::map<uint64_t, Seen> seen;
    uint64_t clock = 0;
    glmflash_graph_stats stats = {};
    uint64_t tick() { return clock == UINT64_MAX ? clock : ++clock; }    // equal ages fall back to key order
    void drop(std::map<uint64_t, Entry>::iterator it) {
        if (it->second.exec) cudaGraphExecDestroy(it->second.exec);
        stats.retained_nodes -= it->second.nodes;
        entries.erase(it);
    }
};

extern "C" int glmflash_graph_policy_default(int bounded, glmflash_graph_policy *out) {
    GF_REQUIRE(out != nullptr, "null argument");
    // upstream's two policies (src/verifier_graph_cache.rs:24-50): capture on first sight either way; the unbounded one
    // keeps at most 32 graphs and clears them all when full
    if (bounded) *out = glmflash_graph_policy{1, 1408, 4194304, 4096, 1};
    else *out = glmflash_graph_policy{0, 32, UINT64_MAX, 0, 1};
    return 0;
}

extern "C" int glmflash_graph_cache_new(const glmflash_graph_policy *policy, glmflash_graph_cache **out) {
    GF_REQUIRE(policy && out, "null argument");
    *out = nullptr;
    GF_REQUIRE(policy->entries >= 1 && policy->after >= 1 && (!policy->bounded || policy->sightings >= 1), "policy: entries, after (and sightings when bounded) must be at least 1");
    glmflash_graph_cache *c = new (std::nothrow) glmflash_graph_cache();
    GF_REQUIRE(c != nullptr, "out of host memory");
    c->policy = *policy;
    *out = c;
    return 0;
}

extern "C" void glmflash_graph_cache_free(glmflash_graph_cache *c) {
    if (!c) return;
    for (auto &kv : c->entries)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    delete c;
}

// Cache::action (src/verifier_graph_cache.rs:134-171)
extern "C" int glmflash_graph_cache_action(glmflash_graph_cache *c, uint64_t key) {
    if (!c) return gf::fail("null argument");
    const uint64_t now = c->tick();
    auto it = c->entries.find(key);
    if (it != c->entries.end()) {
        it->second.used = now;
        c->stats.hits++;
        return GLMFLASH_GRAPH_REPLAY;
    }
    if (!c->policy.bounded) {
        if (c->entries.size() >= c->policy.entries) {
            c->stats.evictions += c->entries.size();
            while (!c->entries.empty()) c->drop(c->entries.begin());
        }
        return GLMFLASH_GRAPH_CAPTURE;
    }
    if (!c->seen.count(key) && c->seen.size() == c->policy.sightings) {
        auto oldest = c->seen.begin();
        for (auto s = c->seen.begin(); s != c->seen.end(); ++s)
            if (s->second.used < oldest->second.used) oldest = s;
        c->seen.erase(oldest);
    }
    auto &s = c->seen[key];
    if (s.count < UINT32_MAX) s.count++;
    s.used = now;
    if (s.count >= c->policy.after) return GLMFLASH_GRAPH_CAPTURE;
    c->stats.eager++;
    return GLMFLASH_GRAPH_EAGER;
}

// Cache::insert (:181-213).  Returns 0 when the graph was retained (the cache owns it now), 1 when it alone exceeds the
// node cap (the caller keeps it: it may launch it once and must destroy it), -1 on a bad argument.
extern "C" int glmflash_graph_cache_insert(glmflash_graph_cache *c, uint64_t key, uint64_t nodes, void *graph_exec) {
    if (!c) return gf::fail("null argument");
    c->stats.captures++;
    if (nodes > c->stats.largest_graph_nodes) c->stats.largest_graph_nodes = nodes;
    c->seen.erase(key);
    if (nodes > c->policy.nodes) {
        c->stats.oversized++;
        return 1;
    }
    auto old = c->entries.find(key);
    if (old != c->entries.end()) c->drop(old);
    while (c->entries.size() >= c->policy.entries || c->stats.retained_nodes > c->policy.nodes - nodes) {
        auto oldest = c->entries.begin();
        for (auto e = c->entries.begin(); e != c->entries.end(); ++e)
            if (e->second.used < oldest->second.used) oldest = e;
        c->drop(oldest);
        c->stats.evictions++;
    }
    c->entries[key] = glmflash_graph_cache::Entry{(cudaGraphExec_t)graph_exec, nodes, c->tick()};
    c->stats.retained_nodes += nodes;
    if (c->entries.size() > c->stats.peak_graphs) c->stats.peak_graphs = c->entries.size();
    if (c->stats.retained_nodes > c->stats.peak_nodes) c->stats.peak_nodes = c->stats.retained_nodes;
    return 0;
}

extern "C" void *glmflash_graph_cache_get(const glmflash_graph_cache *c, uint64_t key) {
    if (!c) return nullptr;
    auto it = c->entries.find(key);
    return it == c->entries.end() ? nullptr : (void *)it->second.exec;
}

extern "C" int glmflash_graph_cache_stats(const glmflash_graph_cache *c, glmflash_graph_stats *out) {
    GF_REQUIRE(c && out, "null argument");
    *out = c->stats;
    out->retained_graphs = c->entries.size();
    out->tracked_sightings = c->seen.size();
    return 0;
}

// The whole step for one window: replay the graph of `key`, or run `enqueue` eagerly, or capture it (relaxed capture on
// the caller's stream), instantiate, launch and retain it -- whatever the policy says.  `enqueue` may only enqueue work
// on the stream it is given (every run function of this library qualifies); it returns 0 or -1.
extern "C" int glmflash_graph_cache_run(glmflash_graph_cache *c, uint64_t key, void *stream, glmflash_enqueue_fn enqueue, void *user) {
    GF_REQUIRE(c && enqueue, "null argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int action = glmflash_graph_cache_action(c, key);
    if (action == GLMFLASH_GRAPH_REPLAY) {
        GF_CUDA(cudaGraphLaunch((cudaGraphExec_t)glmflash_graph_cache_get(c, key), s));
        return 0;
    }
    if (action == GLMFLASH_GRAPH_EAGER) return enqueue(user, stream) ? -1 : 0;
    GF_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
    const int rc = enqueue(user, stream);
    cudaGraph_t graph = nullptr;
    const cudaError_t end = cudaStreamEndCapture(s, &graph);
    if (rc || end != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        return rc ? -1 : gf::fail_cuda(end, "cudaStreamEndCapture");
    }
    size_t nodes = 0;
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphGetNodes(graph, nullptr, &nodes);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return gf::fail_cuda(e, "cudaGraphInstantiate");
    e = cudaGraphLaunch(exec, s);
    if (e != cudaSuccess) {
        cudaGraphExecDestroy(exec);
        return gf::fail_cuda(e, "cudaGraphLaunch");
    }
    if (glmflash_graph_cache_insert(c, key, nodes, exec) == 1) {
        // too large to retain: it has been launched once; destroy it when the stream has run it
        GF_CUDA(cudaStreamSynchronize(s));
        cudaGraphExecDestroy(exec);
    }
    return 0;
}
