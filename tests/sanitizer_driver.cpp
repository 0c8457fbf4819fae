// Host-side fuzz of the cache manager and the session table under AddressSanitizer and
// UndefinedBehaviorSanitizer (built and run by tests/test_manager_sanitizers.py; no CUDA involved).
//
// Compiled together with csrc/manager.cpp and csrc/sessions.cpp.  The handful of C-ABI functions
// that sessions.cpp calls live in api.cu (a CUDA file) in the product; here they are re-stated over
// the same manager functions so that the real manager and session code run under the sanitizers.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include "../combsengine_b200/csrc/manager.hpp"

using namespace cbkv;

extern "C" {
int32_t cbkv_seq_create(cbkv_arena* a, cbkv_seq** out) {
    Seq* s = nullptr;
    int32_t rc = seq_create(reinterpret_cast<Arena*>(a), &s);
    if (rc == CBKV_OK) *out = reinterpret_cast<cbkv_seq*>(s);
    return rc;
}
int32_t cbkv_seq_destroy(cbkv_seq* s) { return seq_destroy(reinterpret_cast<Seq*>(s)); }
int32_t cbkv_popn(cbkv_seq* s, int64_t n, int64_t* popped) { return popn(reinterpret_cast<Seq*>(s), n, popped); }
int64_t cbkv_seq_len(const cbkv_seq* s) { return reinterpret_cast<const Seq*>(s)->seq_len; }
int32_t cbkv_page_stats(const cbkv_seq* s, cbkv_page_stats_t* out) {
    page_stats(reinterpret_cast<const Seq*>(s), 0, out);
    return CBKV_OK;
}
int64_t cbkv_page_bytes(const cbkv_arena* a) {
    const Arena* ar = reinterpret_cast<const Arena*>(a);
    return (int64_t)ar->cfg.num_layers * ar->cfg.page_size * ar->cfg.n_kv_heads * ar->cfg.head_dim * 4;
}
}

#define REQUIRE(cond) do { if (!(cond)) { fprintf(stderr, "sanitizer_driver: %s failed at line %d (%s)\n", #cond, __LINE__, last_error()); return 1; } } while (0)

static int fuzz_manager(uint64_t seed) {
    std::mt19937_64 rng(seed);
    cbkv_config cfg{};
    cfg.num_layers = 3; cfg.n_q_heads = 8; cfg.n_kv_heads = 2; cfg.head_dim = 64; cfg.page_size = 16;
    cfg.dtype = CBKV_F16; cfg.max_seq_len = 900; cfg.num_pages = 200; cfg.sliding_popn_refuses = 0;
    int64_t windows[3] = {0, 64, 0};
    cfg.layer_windows = windows;
    Arena* a = nullptr;
    REQUIRE(arena_create(&cfg, &a) == CBKV_OK);
    std::vector<Seq*> seqs;
    DecodeSplit splits[3] = {DecodeSplit{}, DecodeSplit{25, 4, 5}, DecodeSplit{40, 2, 8}};
    for (int step = 0; step < 3000; step++) {
        const int op = (int)(rng() % 10);
        if (op < 2 && seqs.size() < 12) {
            Seq* s = nullptr;
            REQUIRE(seq_create(a, &s) == CBKV_OK);
            seqs.push_back(s);
        } else if (op < 6 && !seqs.empty()) {  // a step over a random subset, chunk or decode
            std::vector<Seq*> sub;
            std::vector<int64_t> nt, pos;
            const bool decode = rng() % 2;
            for (Seq* s : seqs)
                if (rng() % 2) { sub.push_back(s); nt.push_back(decode ? 1 : 1 + (int64_t)(rng() % 70)); pos.push_back(s->seq_len); }
            const int32_t rc = begin_step(a, sub.data(), nt.data(), pos.data(), (int32_t)sub.size());
            REQUIRE(rc == CBKV_OK || rc == CBKV_ERR_CAPACITY || rc == CBKV_ERR_EXHAUSTED || rc == CBKV_ERR_STATE);
            if (rc == CBKV_OK && !sub.empty()) {
                for (int64_t w : {(int64_t)0, (int64_t)64, (int64_t)17}) {
                    DecodePlan pl;
                    build_decode_plan(*a, w, 1 + (int)(rng() % 300), splits[rng() % 3], &pl);
                    int64_t covered = 0;
                    for (const ItemInfo& it : pl.items) { REQUIRE(it.u_end > it.u_begin); covered += it.u_end - it.u_begin; }
                    REQUIRE(covered == pl.n_units);
                    REQUIRE(pl.segs.back().unit_begin == pl.n_units);
                }
                ChunkPlan cp;
                build_chunk_plan(*a, 16, &cp);
                build_chunk_tile_plan(*a, 32, &cp);
            }
        } else if (op == 6 && !seqs.empty()) {
            Seq* s = seqs[rng() % seqs.size()];
            int64_t popped = 0;
            REQUIRE(popn(s, (int64_t)(rng() % 100), &popped) == CBKV_OK);
        } else if (op == 7 && !seqs.empty() && seqs.size() < 12) {
            Seq* p = seqs[rng() % seqs.size()];
            if (p->seq_len >= 16) {
                Seq* c = nullptr;
                REQUIRE(seq_fork_prefix(p, (int64_t)(1 + rng() % (p->seq_len / 16)) * 16, &c) == CBKV_OK);
                seqs.push_back(c);
            }
        } else if (op == 8 && !seqs.empty()) {
            const size_t i = rng() % seqs.size();
            REQUIRE(seq_destroy(seqs[i]) == CBKV_OK);
            seqs.erase(seqs.begin() + (long)i);
        } else if (op == 9 && !seqs.empty() && rng() % 4 == 0) {
            REQUIRE(reset(seqs[rng() % seqs.size()]) == CBKV_OK);
        }
        // conservation: every page is either free or held, and held pages carry their holders' count
        std::vector<int> held((size_t)a->num_pages, 0);
        for (Seq* s : seqs) for (int64_t p : s->table) held[(size_t)p]++;
        int64_t in_use = 0;
        for (int64_t p = 0; p < a->num_pages; p++) { REQUIRE(held[(size_t)p] == a->refcnt[(size_t)p]); in_use += held[(size_t)p] > 0; }
        REQUIRE(in_use + a->alloc.num_free() == a->num_pages);
    }
    while (!seqs.empty()) { seq_destroy(seqs.back()); seqs.pop_back(); }
    REQUIRE(a->alloc.num_free() == a->num_pages);
    delete a;
    return 0;
}

static int fuzz_sessions(uint64_t seed) {
    std::mt19937_64 rng(seed);
    cbkv_config cfg{};
    cfg.num_layers = 2; cfg.n_q_heads = 4; cfg.n_kv_heads = 2; cfg.head_dim = 64; cfg.page_size = 16;
    cfg.dtype = CBKV_F16; cfg.max_seq_len = 512; cfg.num_pages = 160;
    Arena* a = nullptr;
    REQUIRE(arena_create(&cfg, &a) == CBKV_OK);
    cbkv_sessions* set = nullptr;
    REQUIRE(cbkv_sessions_create(reinterpret_cast<cbkv_arena*>(a), 3, &set) == CBKV_OK);
    const char* keys[5] = {"a", "b", "c", "d\"quoted\"", "e"};
    std::vector<std::vector<uint32_t>> hist(5);
    for (int gen = 0; gen < 400; gen++) {
        const int k = (int)(rng() % 5);
        std::vector<uint32_t> prompt = hist[(size_t)k];
        if (rng() % 3 == 0 && !prompt.empty()) prompt.resize(rng() % prompt.size() + 1);
        for (int i = 0, n = 1 + (int)(rng() % 40); i < n; i++) prompt.push_back((uint32_t)(rng() % 50));
        if (prompt.size() > 300) prompt.resize(300);
        cbkv_seq* seq = nullptr;
        int64_t lcp = 0;
        REQUIRE(cbkv_sessions_acquire(set, keys[k], prompt.data(), (int64_t)prompt.size(), 1, &seq, &lcp) == CBKV_OK);
        REQUIRE(lcp >= 0 && lcp < (int64_t)prompt.size() && cbkv_seq_len(seq) == lcp);
        // "prefill" the rest of the prompt, then a few decode steps with one speculative round
        Seq* s = reinterpret_cast<Seq*>(seq);
        int64_t nt = (int64_t)prompt.size() - lcp, pos = lcp;
        REQUIRE(begin_step(a, &s, &nt, &pos, 1) == CBKV_OK);
        const uint32_t draft[3] = {1, 2, 3}, argmax[4] = {1, 2, 9, 4};
        nt = 4; pos = s->seq_len;
        if (s->seq_len + 4 <= cfg.max_seq_len && begin_step(a, &s, &nt, &pos, 1) == CBKV_OK) {
            int32_t accepted = -1; uint32_t corr = 0;
            REQUIRE(cbkv_spec_verify_rollback(seq, draft, argmax, 3, &accepted, &corr) == CBKV_OK);
            REQUIRE(accepted == 2 && corr == 9);
            prompt.push_back(7); prompt.push_back(1); prompt.push_back(2);  // next + the accepted drafts
        }
        REQUIRE((int64_t)prompt.size() == cbkv_seq_len(seq));
        REQUIRE(cbkv_sessions_release(set, keys[k], seq, prompt.data(), (int64_t)prompt.size(), 1) == CBKV_OK);
        hist[(size_t)k] = prompt;
        REQUIRE(cbkv_sessions_count(set) <= 3);
        char buf[64];
        const int64_t need = cbkv_sessions_stats_json(set, buf, sizeof buf);  // truncation must stay in bounds
        REQUIRE(need > 0);
        std::string full((size_t)need + 1, '\0');
        REQUIRE(cbkv_sessions_stats_json(set, full.data(), need + 1) == need);
        for (int j = 0; j < 5; j++) if (cbkv_sessions_history_len(set, keys[j]) < 0) hist[(size_t)j].clear();  // evicted
    }
    int64_t removed = 0;
    REQUIRE(cbkv_sessions_clear(set, &removed) == CBKV_OK);
    REQUIRE(cbkv_sessions_destroy(set) == CBKV_OK);
    REQUIRE(a->alloc.num_free() == a->num_pages);
    delete a;
    return 0;
}

int main(int argc, char** argv) {
    const uint64_t seed = argc > 1 ? strtoull(argv[1], nullptr, 10) : 1;
    if (int rc = fuzz_manager(seed)) return rc;
    if (int rc = fuzz_sessions(seed + 1000)) return rc;
    printf("sanitizer_driver ok (seed %llu)\n", (unsigned long long)seed);
    return 0;
}
