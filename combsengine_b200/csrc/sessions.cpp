// Session table and rollback helpers: the callers that drive allocate / popn / reuse on the
// paged cache.  Host code only; every cache operation goes through the C ABI of this library.
//
// Reference: combs-runtime/src/engine.rs
//   SessionSet (take / put with LRU eviction / clear_all)            :266-314
//   longest-common-prefix reuse at the start of a generation         :1257-1287
//   speculative-verify acceptance and rollback                       :1476-1500
//   session snapshot after a generation                              :1541-1568
// and the "kv" object of GET /v1/stats, combs-cli/src/serve.rs:146-166,197-208.
//
// The reference gives every session a cache with a private arena; here the sessions are
// sequences of one shared arena, so dropping a session returns its pages to the common
// free-list at once.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "manager.hpp"

using namespace cbkv;

namespace {

struct Session {
    std::vector<uint32_t> history;  // prompt + decoded tokens: exactly what the cache holds
    cbkv_seq* seq = nullptr;
    uint64_t last_used = 0;
};

struct SessionSet {
    cbkv_arena* arena = nullptr;
    int32_t max_sessions = 4;  // MAX_SESSIONS, engine.rs:243
    std::map<std::string, Session> map;
    uint64_t tick = 0, evictions = 0;
};

size_t common_prefix(const std::vector<uint32_t>& a, const uint32_t* b, int64_t nb) {  // engine.rs:386-388
    size_t n = 0;
    while (n < a.size() && (int64_t)n < nb && a[n] == b[n]) n++;
    return n;
}

void json_string(std::string& out, const std::string& s) {
    out += '"';
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { out += '\\'; out += (char)c; }
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out += (char)c;
    }
    out += '"';
}

}  // namespace

extern "C" {

int32_t cbkv_sessions_create(cbkv_arena* arena, int32_t max_sessions, cbkv_sessions** out) {
    return fenced([&]() -> int32_t {
    if (!arena || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (max_sessions < 0) { set_error("max_sessions must be >= 0 (0 = the default of 4)"); return CBKV_ERR_ARG; }
    auto* s = new SessionSet();
    s->arena = arena;
    if (max_sessions > 0) s->max_sessions = max_sessions;
    *out = reinterpret_cast<cbkv_sessions*>(s);
    return CBKV_OK;
    });
}

int32_t cbkv_sessions_destroy(cbkv_sessions* set) {
    return fenced([&]() -> int32_t {
    auto* s = reinterpret_cast<SessionSet*>(set);
    if (!s) return CBKV_OK;
    for (auto& kv : s->map) cbkv_seq_destroy(kv.second.seq);
    delete s;
    return CBKV_OK;
    });
}

int32_t cbkv_sessions_acquire(cbkv_sessions* set, const char* key, const uint32_t* prompt, int64_t n_prompt,
                              int32_t reuse, cbkv_seq** seq_out, int64_t* lcp_out) {
    return fenced([&]() -> int32_t {
    auto* s = reinterpret_cast<SessionSet*>(set);
    if (!s || !seq_out || !lcp_out || (n_prompt > 0 && !prompt)) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (n_prompt < 1) { set_error("empty prompt"); return CBKV_ERR_ARG; }  // engine.rs:1235-1237
    *lcp_out = 0;
    *seq_out = nullptr;
    cbkv_seq* seq = nullptr;
    if (reuse) {
        auto it = s->map.find(key ? key : "");
        if (it != s->map.end()) {  // sessions.take, engine.rs:1264
            Session old = std::move(it->second);
            s->map.erase(it);
            // capped at len - 1: the last position's logits are always needed (engine.rs:1257-1260)
            const int64_t shared = std::min<int64_t>((int64_t)common_prefix(old.history, prompt, n_prompt), n_prompt - 1);
            if (shared > 0) {
                const int64_t need = (int64_t)old.history.size() - shared;
                int64_t popped = 0;
                int32_t rc = cbkv_popn(old.seq, need, &popped);
                if (rc == CBKV_OK && popped == need) {  // engine.rs:1270-1274
                    seq = old.seq;
                    *lcp_out = shared;
                }
            }
            // no shared prefix, or a rollback the cache refuses (sliding layers past eviction, a cut
            // inside a shared page): never continue on divergent state, start fresh (engine.rs:1275-1284)
            if (!seq) cbkv_seq_destroy(old.seq);
        }
    }
    if (!seq) {
        int32_t rc = cbkv_seq_create(s->arena, &seq);
        if (rc) return rc;
    }
    *seq_out = seq;
    return CBKV_OK;
    });
}

int32_t cbkv_sessions_release(cbkv_sessions* set, const char* key, cbkv_seq* seq, const uint32_t* history,
                              int64_t n_history, int32_t reuse) {
    return fenced([&]() -> int32_t {
    auto* s = reinterpret_cast<SessionSet*>(set);
    if (!s || !seq || (n_history > 0 && !history)) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (!reuse) return cbkv_seq_destroy(seq);  // the cache of a request outside the session table is dropped
    if (cbkv_seq_len(seq) != n_history) {      // history must mirror the cache exactly (engine.rs:1549-1551)
        set_error("session history (" + std::to_string(n_history) + " tokens) does not mirror the cache (" +
                  std::to_string(cbkv_seq_len(seq)) + ")");
        return CBKV_ERR_STATE;
    }
    const std::string k = key ? key : "";
    auto it = s->map.find(k);
    if (it != s->map.end()) {  // HashMap::insert replaces, the old value is dropped
        if (it->second.seq != seq) cbkv_seq_destroy(it->second.seq);
        s->map.erase(it);
    }
    Session ns;
    ns.history.assign(history, history + n_history);
    ns.seq = seq;
    ns.last_used = ++s->tick;  // engine.rs:297-299
    s->map.emplace(k, std::move(ns));
    if ((int64_t)s->map.size() > s->max_sessions) {  // engine.rs:300-311
        auto oldest = s->map.begin();
        for (auto i = s->map.begin(); i != s->map.end(); ++i)
            if (i->second.last_used < oldest->second.last_used) oldest = i;
        cbkv_seq_destroy(oldest->second.seq);
        s->map.erase(oldest);
        s->evictions++;
    }
    return CBKV_OK;
    });
}

int32_t cbkv_sessions_clear(cbkv_sessions* set, int64_t* removed) {
    return fenced([&]() -> int32_t {  // clear_all, engine.rs:287-291
    auto* s = reinterpret_cast<SessionSet*>(set);
    if (!s) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (removed) *removed = (int64_t)s->map.size();
    for (auto& kv : s->map) cbkv_seq_destroy(kv.second.seq);
    s->map.clear();
    return CBKV_OK;
    });
}

int64_t cbkv_sessions_count(const cbkv_sessions* set) {
    return fenced64([&]() -> int64_t {
    auto* s = reinterpret_cast<const SessionSet*>(set);
    return s ? (int64_t)s->map.size() : 0;
    });
}

int64_t cbkv_sessions_evictions(const cbkv_sessions* set) {
    return fenced64([&]() -> int64_t {
    auto* s = reinterpret_cast<const SessionSet*>(set);
    return s ? (int64_t)s->evictions : 0;
    });
}

int64_t cbkv_sessions_history_len(const cbkv_sessions* set, const char* key) {
    return fenced64([&]() -> int64_t {
    auto* s = reinterpret_cast<const SessionSet*>(set);
    if (!s) return -1;
    auto it = s->map.find(key ? key : "");
    return it == s->map.end() ? -1 : (int64_t)it->second.history.size();
    });
}

int32_t cbkv_spec_verify_rollback(cbkv_seq* seq, const uint32_t* draft, const uint32_t* argmax, int32_t k,
                                  int32_t* accepted_out, uint32_t* correction_out) {
    return fenced([&]() -> int32_t {
    if (!seq || !draft || !argmax || !accepted_out || !correction_out || k < 0) { set_error("null argument"); return CBKV_ERR_ARG; }
    int32_t accepted = 0;
    while (accepted < k && argmax[accepted] == draft[accepted]) accepted++;  // engine.rs:1476-1479
    *accepted_out = accepted;
    *correction_out = argmax[std::min(accepted, k)];                          // engine.rs:1480
    const int64_t unwanted = k - accepted;
    if (unwanted > 0) {                                                        // engine.rs:1484-1493
        int64_t popped = 0;
        int32_t rc = cbkv_popn(seq, unwanted, &popped);
        if (rc) return rc;
        if (popped != unwanted) {
            set_error("speculative rollback popped " + std::to_string(popped) + " of " + std::to_string(unwanted) + " rows");
            return CBKV_ERR_STATE;
        }
    }
    return CBKV_OK;
    });
}

int64_t cbkv_sessions_stats_json(const cbkv_sessions* set, char* buf, int64_t cap) {
    return fenced64([&]() -> int64_t {
    auto* s = reinterpret_cast<const SessionSet*>(set);
    if (!s) { set_error("null argument"); return CBKV_ERR_ARG; }
    const Arena* a = reinterpret_cast<const Arena*>(s->arena);
    const int64_t page_bytes = cbkv_page_bytes(s->arena);
    std::string o = "{";
    auto num = [&](const char* k, long long v, bool comma = true) { o += '"'; o += k; o += "\":"; o += std::to_string(v); if (comma) o += ','; };
    o += "\"kind\":\"paged\",\"quantized\":";
    o += a->cfg.quantize_kv ? "true," : "false,";
    num("max_seq_len", a->cfg.max_seq_len);
    num("page_size", a->cfg.page_size);
    num("page_bytes", page_bytes);
    num("arena_bytes", a->num_pages * page_bytes);
    num("bytes_per_token", page_bytes / std::max(1, a->cfg.page_size));
    num("max_sessions", s->max_sessions);
    num("evictions", (long long)s->evictions);
    o += "\"sessions\":[";
    bool first = true;
    for (const auto& kv : s->map) {
        if (!first) o += ',';
        first = false;
        cbkv_page_stats_t st{};
        cbkv_page_stats(kv.second.seq, &st);
        o += "{\"id\":";
        json_string(o, kv.first.empty() ? "(anonymous)" : kv.first);  // engine.rs:1168-1172
        o += ',';
        num("history_tokens", (long long)kv.second.history.size());
        o += "\"pages\":{";
        num("used", st.pages_used); num("free", st.pages_free); num("total", st.num_pages); num("page_size", st.page_size);
        num("seq_len", st.seq_len); num("kv_bytes", st.pages_used * page_bytes);
        num("layers_materialized", st.layers_materialized); num("layers_total", st.layers_total);
        num("layers_sliding", st.layers_sliding, false);
        o += "}}";
    }
    o += "]}";
    if (buf && cap > 0) {
        const size_t n = std::min<size_t>(o.size(), (size_t)cap - 1);
        memcpy(buf, o.data(), n);
        buf[n] = 0;
    }
    return (int64_t)o.size();
    });
}
}  // extern "C"
