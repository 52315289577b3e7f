// cache2 page-table manager: the host-side producer of the page tables the paged kernels consume.
//
// The reference ships only the design of cache2 (docs/plans/04-kv-cache.md:40-51 "Radix trie (in RAM)":
// keys are token-id sequences, nodes own pages of global KV, page = 16..512 tokens, default 256 --
// crates/sg-cache/src/lib.rs:9-13 holds just those constants).  This file builds step 1 of that plan
// ("pure in-memory trie + lookup/insert/split", 04-kv-cache.md:113) in its page-aligned form, plus the
// physical page pool: a trie whose edges are whole pages of token ids, reference-counted physical
// pages, prefix sharing between sequences, and least-recently-used reclaim of cached pages that no
// live sequence holds.  NVMe persistence, tail snapshots and the cost-aware eviction score of that
// document are outside the attention path and not built.  Pure host code: no CUDA call in here.
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/sgattn.h"
#include "sgb_kernels.h"

namespace {

struct Node {
    std::vector<int32_t> tokens;  // exactly page_tokens ids: the edge from the parent
    uint32_t phys = 0;            // physical page holding their K/V
    Node* parent = nullptr;
    std::map<std::vector<int32_t>, std::unique_ptr<Node>> children;
    uint32_t live = 0;            // sequences currently holding this page
    uint64_t last_use = 0;
    uint64_t lru_key = 0;  // last_use under which the node sits in the reclaim set
    bool in_lru = false;   // true while live == 0 && children.empty()
};

struct Sequence {
    // Logical page i lives in physical page phys[i]; node[i] is the trie node this sequence holds for
    // it, or NULL while the page is private to the sequence.
    std::vector<uint32_t> phys;
    std::vector<Node*> node;
};

}  // namespace

struct sgb_cache2 {
    uint32_t page_tokens, pool_pages;
    Node root;
    std::vector<uint32_t> free_pages;
    std::set<std::pair<uint64_t, Node*>> lru;  // reclaimable leaves ordered by last use, oldest first
    std::unordered_map<uint64_t, Sequence> seqs;
    uint64_t next_seq = 1, clock = 0;
    uint64_t hits = 0, misses = 0, evictions = 0;

    void lru_update(Node* n)
    {
        const bool evictable = n != &root && n->live == 0 && n->children.empty();
        if (n->in_lru) {
            lru.erase({n->lru_key, n});
            n->in_lru = false;
        }
        if (evictable) {
            n->lru_key = n->last_use;
            lru.insert({n->lru_key, n});
            n->in_lru = true;
        }
    }
    // A free physical page, reclaiming the least recently used cached leaf if the pool is empty.
    bool take_page(uint32_t* out)
    {
        if (free_pages.empty()) {
            if (lru.empty()) return false;
            Node* victim = lru.begin()->second;
            lru.erase(lru.begin());
            victim->in_lru = false;
            Node* parent = victim->parent;
            free_pages.push_back(victim->phys);
            parent->children.erase(victim->tokens);  // destroys victim
            evictions++;
            lru_update(parent);
        }
        *out = free_pages.back();
        free_pages.pop_back();
        return true;
    }
};

extern "C" {

int sgb_cache2_create(uint32_t page_tokens, uint32_t pool_pages, sgb_cache2** out)
{
    if (!out) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_create: out is NULL");
    if (page_tokens < 16 || page_tokens > 512 || (page_tokens & (page_tokens - 1)))
        return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_create: page size must be a power of two in 16..512 tokens");
    if (pool_pages == 0) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_create: empty pool");
    sgb_cache2* c = new sgb_cache2();
    c->page_tokens = page_tokens;
    c->pool_pages = pool_pages;
    for (uint32_t p = pool_pages; p-- > 0;) c->free_pages.push_back(p);  // page 0 is handed out first
    *out = c;
    return SGB_OK;
}

void sgb_cache2_destroy(sgb_cache2* c) { delete c; }

int sgb_cache2_lookup(sgb_cache2* c, const int32_t* tokens, uint64_t n_tokens, uint64_t* matched_tokens)
{
    if (!c || (!tokens && n_tokens) || !matched_tokens) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_lookup: NULL argument");
    Node* at = &c->root;
    uint64_t pages = 0;
    const uint32_t P = c->page_tokens;
    while ((pages + 1) * P <= n_tokens) {
        std::vector<int32_t> key(tokens + pages * P, tokens + (pages + 1) * P);
        auto it = at->children.find(key);
        if (it == at->children.end()) break;
        at = it->second.get();
        pages++;
    }
    *matched_tokens = pages * P;
    return SGB_OK;
}

int sgb_cache2_acquire(sgb_cache2* c, const int32_t* tokens, uint64_t n_tokens, uint64_t capacity_tokens, uint32_t* table,
                       uint32_t table_capacity, uint32_t* n_pages, uint64_t* reused_tokens, uint64_t* seq)
{
    if (!c || (!tokens && n_tokens) || !table || !n_pages || !reused_tokens || !seq)
        return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_acquire: NULL argument");
    const uint32_t P = c->page_tokens;
    if (capacity_tokens < n_tokens) capacity_tokens = n_tokens;
    const uint64_t need = (capacity_tokens + P - 1) / P;
    if (need > table_capacity) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_acquire: page table too small for the sequence");
    Sequence s;
    // 1. longest page-aligned prefix already cached: share those pages.  Only pages that the given
    //    tokens fill completely are shared, so the page a sequence appends into is always private.
    Node* at = &c->root;
    while ((s.node.size() + 1) * (uint64_t)P <= n_tokens) {
        std::vector<int32_t> key(tokens + s.node.size() * P, tokens + (s.node.size() + 1) * P);
        auto it = at->children.find(key);
        if (it == at->children.end()) break;
        at = it->second.get();
        s.node.push_back(at);
        s.phys.push_back(at->phys);
    }
    const size_t n_shared = s.node.size();
    for (Node* n : s.node) {  // pin before reclaiming, so the prefix cannot be evicted from under us
        n->live++;
        n->last_use = ++c->clock;
        c->lru_update(n);
    }
    // 2. private pages for the rest
    while (s.phys.size() < need) {
        uint32_t p;
        if (!c->take_page(&p)) {
            for (size_t i = n_shared; i < s.phys.size(); i++) c->free_pages.push_back(s.phys[i]);
            for (size_t i = n_shared; i-- > 0;) {
                s.node[i]->live--;
                c->lru_update(s.node[i]);
            }
            return sgb::set_last_error(SGB_ERR_STATE, "sgb_cache2_acquire: the page pool is exhausted (every page is held by a live sequence)");
        }
        s.phys.push_back(p);
        s.node.push_back(nullptr);
    }
    for (size_t i = 0; i < s.phys.size(); i++) table[i] = s.phys[i];
    *n_pages = (uint32_t)need;
    *reused_tokens = n_shared * (uint64_t)P;
    if (n_shared) c->hits++; else c->misses++;
    *seq = c->next_seq++;
    c->seqs[*seq] = std::move(s);
    return SGB_OK;
}

int sgb_cache2_commit(sgb_cache2* c, uint64_t seq, const int32_t* tokens, uint64_t n_tokens)
{
    if (!c || (!tokens && n_tokens)) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_commit: NULL argument");
    auto it = c->seqs.find(seq);
    if (it == c->seqs.end()) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_commit: unknown sequence");
    Sequence& s = it->second;
    const uint32_t P = c->page_tokens;
    Node* at = &c->root;
    // Every private page the tokens fill completely becomes a trie node (insert on commit,
    // 04-kv-cache.md:47-48).  Where an equal page was committed by another sequence meanwhile, ours stays
    // private and the walk goes on below the existing node: the K/V of a page depends only on the tokens
    // up to its end, so deeper pages of this sequence are valid continuations of that node.
    for (size_t i = 0; i < s.phys.size() && (i + 1) * (uint64_t)P <= n_tokens; i++) {
        if (s.node[i]) {
            at = s.node[i];
            continue;
        }
        std::vector<int32_t> key(tokens + i * P, tokens + (i + 1) * P);
        auto found = at->children.find(key);
        if (found != at->children.end()) {
            at = found->second.get();
            continue;
        }
        std::unique_ptr<Node> n(new Node());
        n->tokens = key;
        n->phys = s.phys[i];
        n->parent = at;
        n->live = 1;
        n->last_use = ++c->clock;
        Node* raw = n.get();
        at->children[key] = std::move(n);
        c->lru_update(at);  // the parent is no longer a leaf
        s.node[i] = raw;
        at = raw;
    }
    return SGB_OK;
}

int sgb_cache2_release(sgb_cache2* c, uint64_t seq)
{
    if (!c) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_release: NULL argument");
    auto it = c->seqs.find(seq);
    if (it == c->seqs.end()) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_release: unknown sequence");
    Sequence& s = it->second;
    // deepest first, so a chain of now-idle pages enters the reclaim list leaf-most first
    for (size_t i = s.phys.size(); i-- > 0;) {
        if (s.node[i]) {
            s.node[i]->live--;
            c->lru_update(s.node[i]);
        } else {
            c->free_pages.push_back(s.phys[i]);
        }
    }
    c->seqs.erase(it);
    return SGB_OK;
}

int sgb_cache2_stats(const sgb_cache2* c, sgb_cache2_stats_t* out)
{
    if (!c || !out) return sgb::set_last_error(SGB_ERR_VALIDATION, "sgb_cache2_stats: NULL argument");
    out->page_tokens = c->page_tokens;
    out->pool_pages = c->pool_pages;
    out->free_pages = (uint32_t)c->free_pages.size();
    out->reclaimable_pages = (uint32_t)c->lru.size();
    out->live_sequences = (uint32_t)c->seqs.size();
    out->reserved = 0;
    out->hits = c->hits;
    out->misses = c->misses;
    out->evictions = c->evictions;
    return SGB_OK;
}

}  // extern "C"
