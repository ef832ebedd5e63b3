// Host-side runtime of the engine, in plain C++ behind a C interface (loaded
// with ctypes; no CUDA in here): the cache manager (page pools, block tables per
// request and group, state slots) and the packing of a step's batch into the
// one array of 32-bit integers that travels to the device.
//
// Pages: the free list starts as 0..n-1, pages are taken from its front and given
// back at its back, so reuse is first-in first-out (src/block_manager.cc:17-23,
// 47-50,61-62).  reserve grows a request to a token count or changes nothing
// (src/block_manager.cc:32-53); release gives everything back and may be called
// twice (src/block_manager.cc:55-64).  A group with a window gives a page back as
// soon as no later query can see any of its positions.  The flattening of a batch
// and its checks follow src/model_batch.cc:34-125,127-204.
//
// Every entry point returns 0 or a positive value on success and a negative
// RT_* code on failure; chibi_rt_error() then holds the message (per thread).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#define RT_API extern "C" __attribute__((visibility("default")))

namespace {

enum : int {
    RT_CAPACITY_EXHAUSTED = -1,
    RT_INVALID_RELEASE = -2,
    RT_UNKNOWN_REQUEST = -3,
    RT_DUPLICATE_REQUEST = -4,
    RT_INVALID_RESERVATION = -5,
    RT_INVALID_COMMIT = -6,
    RT_INVALID_CONFIGURATION = -7,
    RT_INVARIANT = -8,
    RT_BATCH = -9,
    RT_BUFFER_TOO_SMALL = -10,
};

thread_local std::string g_error;

int fail(int code, const std::string& message)
{
    g_error = message;
    return code;
}

std::string str(long long v) { return std::to_string(v); }

// ------------------------------------------------------------------ pools
class PagePool {
public:
    explicit PagePool(int num_pages) : held_(num_pages, 0)
    {
        for (int p = 0; p < num_pages; ++p)
            free_.push_back(p);
    }
    int num_pages() const { return static_cast<int>(held_.size()); }
    int free_count() const { return static_cast<int>(free_.size()); }
    // `count` pages from the front of the free list, appended to `out`; or nothing
    int take(int count, std::vector<int>* out)
    {
        if (count > free_count())
            return fail(RT_CAPACITY_EXHAUSTED, str(count) + " pages wanted, " + str(free_count()) + " free");
        for (int i = 0; i < count; ++i) {
            const int p = free_.front();
            free_.pop_front();
            held_[p] = 1;
            out->push_back(p);
        }
        return 0;
    }
    int give(int page)
    {
        if (page < 0 || page >= num_pages() || !held_[page])
            return fail(RT_INVALID_RELEASE, "page " + str(page) + " is not held");
        held_[page] = 0;
        free_.push_back(page);
        return 0;
    }
    const std::deque<int>& free_list() const { return free_; }

private:
    std::deque<int> free_;
    std::vector<char> held_;
};

// State slots, lowest free index first.
class SlotPool {
public:
    explicit SlotPool(int n) : held_(n, 0) {}
    int num_slots() const { return static_cast<int>(held_.size()); }
    int free_count() const { return num_slots() - used_; }
    int take()
    {
        for (int s = 0; s < num_slots(); ++s)
            if (!held_[s]) {
                held_[s] = 1;
                ++used_;
                return s;
            }
        return fail(RT_CAPACITY_EXHAUSTED, "no state slot is free");
    }
    int give(int slot)
    {
        if (slot < 0 || slot >= num_slots() || !held_[slot])
            return fail(RT_INVALID_RELEASE, "state slot " + str(slot) + " is not held");
        held_[slot] = 0;
        --used_;
        return 0;
    }

private:
    std::vector<char> held_;
    int used_ = 0;
};

int pages_for(int tokens, int page_size) { return tokens <= 0 ? 0 : 1 + (tokens - 1) / page_size; }

// Lowest logical block that a query at position >= length can still see: such a query
// sees keys at positions > its own - window, so positions below length - window + 1 are dead.
int first_needed_block(int length, int window, int page_size)
{
    if (window < 0)
        return 0;
    const int first_pos = std::max(0, length - window + 1);
    return first_pos / page_size;
}

// ------------------------------------------------------------------ cache manager
struct Group {
    int page_size, num_pages, window /* -1: none */, max_blocks /* 0: no limit */;
};

struct Update {
    int row, index, page;
};

struct Request {
    int length = 0;      // tokens whose keys are stored (committed)
    int settled = 0;     // length up to which window pages have been given back (<= length)
    int reserved = 0;    // tokens that the tables have room for
    int slot = -1;
    std::vector<std::vector<int>> tables;   // per group: logical block -> page, -1 once the window has passed it
};

class CacheManager {
public:
    CacheManager(std::vector<Group> groups, int max_requests) : groups_(std::move(groups)), slots_(max_requests)
    {
        for (const Group& g : groups_) {
            pools_.emplace_back(g.num_pages);
            updates_.emplace_back();
        }
    }
    int num_groups() const { return static_cast<int>(groups_.size()); }
    const Group& group(int g) const { return groups_[g]; }
    const PagePool& pool(int g) const { return pools_[g]; }
    const SlotPool& slots() const { return slots_; }
    size_t count() const { return requests_.size(); }
    const std::unordered_map<long long, Request>& requests() const { return requests_; }

    Request* find(long long id)
    {
        auto it = requests_.find(id);
        return it == requests_.end() ? nullptr : &it->second;
    }
    int admit(long long id)
    {
        if (requests_.count(id))
            return fail(RT_DUPLICATE_REQUEST, "request is already admitted");
        const int slot = slots_.take();
        if (slot < 0)
            return slot;
        Request r;
        r.slot = slot;
        r.tables.resize(groups_.size());
        requests_.emplace(id, std::move(r));
        return slot;
    }
    // Make room for the request to hold `tokens` tokens, in every group, or change nothing.
    int reserve(long long id, int tokens)
    {
        if (tokens <= 0)
            return fail(RT_INVALID_RESERVATION, "a reservation needs at least one token");
        Request* r = find(id);
        if (!r)
            return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
        if (tokens <= r->reserved)
            return 0;
        std::vector<int> need(groups_.size());
        for (size_t g = 0; g < groups_.size(); ++g) {
            need[g] = pages_for(tokens, groups_[g].page_size) - static_cast<int>(r->tables[g].size());
            if (need[g] > pools_[g].free_count())
                return fail(RT_CAPACITY_EXHAUSTED, "group " + str(g) + ": " + str(need[g]) + " pages wanted, "
                                                       + str(pools_[g].free_count()) + " free");
            const int limit = groups_[g].max_blocks;
            if (need[g] > 0 && limit && static_cast<int>(r->tables[g].size()) + need[g] > limit)
                return fail(RT_INVALID_RESERVATION, "group " + str(g) + ": "
                                                        + str((long long)r->tables[g].size() + need[g])
                                                        + " blocks exceed the table's " + str(limit));
        }
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (need[g] <= 0)
                continue;
            std::vector<int> pages;
            pools_[g].take(need[g], &pages);
            for (int page : pages) {
                updates_[g].push_back({ r->slot, static_cast<int>(r->tables[g].size()), page });
                r->tables[g].push_back(page);
            }
        }
        r->reserved = std::max(r->reserved, tokens);
        return 0;
    }
    // The request now holds `new_length` tokens; pages that its windows have passed go back.
    // With `hold` nothing is given back yet: the length can still be taken back by rollback()
    // (a step whose result turns out to be unusable), until settle() makes it final.  The
    // reference opens and closes a transaction on its state around every batch for the same
    // purpose (src/model_state.h:86-99, src/qwen/qwen3_5_model_state.cc:284-370).
    int commit(long long id, int new_length, bool hold = false)
    {
        Request* r = find(id);
        if (!r)
            return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
        if (new_length < r->length || new_length > r->reserved)
            return fail(RT_INVALID_COMMIT, "length " + str(r->length) + " -> " + str(new_length) + ", reserved "
                                               + str(r->reserved));
        r->length = new_length;
        return hold ? 0 : settle(id);
    }
    // Give back what the windows have passed at the current length.
    int settle(long long id)
    {
        Request* r = find(id);
        if (!r)
            return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
        r->settled = r->length;
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (groups_[g].window < 0)
                continue;
            std::vector<int>& table = r->tables[g];
            const int dead = std::min(first_needed_block(r->length, groups_[g].window, groups_[g].page_size),
                                      static_cast<int>(table.size()));
            for (int i = 0; i < dead; ++i) {
                if (table[i] >= 0) {
                    pools_[g].give(table[i]);
                    updates_[g].push_back({ r->slot, i, -1 });
                    table[i] = -1;
                }
            }
        }
        return 0;
    }
    // Take a held commit back: the request holds `old_length` tokens again.  Pages stay
    // reserved, so the same tokens can be run again at the same places.
    int rollback(long long id, int old_length)
    {
        Request* r = find(id);
        if (!r)
            return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
        if (old_length < r->settled || old_length > r->length)
            return fail(RT_INVALID_COMMIT, "rollback to " + str(old_length) + ": settled " + str(r->settled)
                                               + ", length " + str(r->length));
        r->length = old_length;
        return 0;
    }
    int release(long long id)
    {
        auto it = requests_.find(id);
        if (it == requests_.end())
            return 0;
        Request& r = it->second;
        for (size_t g = 0; g < groups_.size(); ++g)
            for (int page : r.tables[g])
                if (page >= 0)
                    pools_[g].give(page);
        slots_.give(r.slot);
        requests_.erase(it);
        return 0;
    }
    // Block-table changes since the last call, for the mirror on the device: at most one per
    // (row, block), the latest (they are applied in parallel), in the order of first change.
    std::vector<Update> drain(int g)
    {
        std::vector<Update> out;
        std::unordered_map<long long, size_t> where;
        for (const Update& u : updates_[g]) {
            const long long key = (static_cast<long long>(u.row) << 32) | static_cast<uint32_t>(u.index);
            auto it = where.find(key);
            if (it == where.end()) {
                where.emplace(key, out.size());
                out.push_back(u);
            } else {
                out[it->second].page = u.page;
            }
        }
        updates_[g].clear();
        return out;
    }
    size_t pending_updates(int g) const { return updates_[g].size(); }
    int check() const
    {
        for (size_t g = 0; g < groups_.size(); ++g) {
            std::unordered_set<int> held;
            size_t held_count = 0;
            for (const auto& kv : requests_)
                for (int page : kv.second.tables[g])
                    if (page >= 0) {
                        ++held_count;
                        held.insert(page);
                    }
            if (held.size() != held_count)
                return fail(RT_INVARIANT, "group " + str(g) + ": a page is held twice");
            std::unordered_set<int> free;
            for (int page : pools_[g].free_list()) {
                if (!free.insert(page).second || held.count(page))
                    return fail(RT_INVARIANT, "group " + str(g) + ": free list and tables overlap");
            }
            if (static_cast<int>(free.size() + held.size()) != pools_[g].num_pages())
                return fail(RT_INVARIANT, "group " + str(g) + ": "
                                              + str(pools_[g].num_pages() - (long long)free.size() - (long long)held.size())
                                              + " pages lost");
        }
        std::unordered_set<int> used;
        for (const auto& kv : requests_)
            if (!used.insert(kv.second.slot).second)
                return fail(RT_INVARIANT, "a state slot is held twice");
        if (static_cast<int>(used.size()) + slots_.free_count() != slots_.num_slots())
            return fail(RT_INVARIANT, "a state slot is lost");
        return 0;
    }

private:
    std::vector<Group> groups_;
    std::vector<PagePool> pools_;
    SlotPool slots_;
    std::unordered_map<long long, Request> requests_;
    std::vector<std::vector<Update>> updates_;
};

int align4(int n) { return (n + 3) & ~3; }

} // namespace

// ------------------------------------------------------------------ C interface
RT_API const char* chibi_rt_error() { return g_error.c_str(); }

RT_API void* chibi_pool_new(int num_pages)
{
    if (num_pages <= 0) {
        fail(RT_INVALID_CONFIGURATION, "a page pool needs at least one page");
        return nullptr;
    }
    return new PagePool(num_pages);
}
RT_API void chibi_pool_delete(void* pool) { delete static_cast<PagePool*>(pool); }
RT_API int chibi_pool_free_count(void* pool) { return static_cast<PagePool*>(pool)->free_count(); }
RT_API int chibi_pool_take(void* pool, int count, int* out)
{
    std::vector<int> pages;
    const int st = static_cast<PagePool*>(pool)->take(count, &pages);
    if (st < 0)
        return st;
    std::copy(pages.begin(), pages.end(), out);
    return count;
}
RT_API int chibi_pool_give(void* pool, int page) { return static_cast<PagePool*>(pool)->give(page); }

RT_API void* chibi_cache_new(int num_groups, const int* page_size, const int* num_pages, const int* window,
                             const int* max_blocks, int max_requests)
{
    if (max_requests <= 0) {
        fail(RT_INVALID_CONFIGURATION, "max_requests must be positive");
        return nullptr;
    }
    std::vector<Group> groups;
    for (int g = 0; g < num_groups; ++g) {
        if (page_size[g] <= 0 || num_pages[g] <= 0) {
            fail(RT_INVALID_CONFIGURATION, "a page pool needs at least one page of at least one token");
            return nullptr;
        }
        groups.push_back({ page_size[g], num_pages[g], window[g], max_blocks[g] });
    }
    return new CacheManager(std::move(groups), max_requests);
}
RT_API void chibi_cache_delete(void* cache) { delete static_cast<CacheManager*>(cache); }
RT_API int chibi_cache_admit(void* cache, long long id) { return static_cast<CacheManager*>(cache)->admit(id); }
RT_API int chibi_cache_has(void* cache, long long id) { return static_cast<CacheManager*>(cache)->find(id) ? 1 : 0; }
RT_API int chibi_cache_count(void* cache) { return static_cast<int>(static_cast<CacheManager*>(cache)->count()); }
// out: length, reserved, state slot
RT_API int chibi_cache_info(void* cache, long long id, int* out)
{
    const Request* r = static_cast<CacheManager*>(cache)->find(id);
    if (!r)
        return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
    out[0] = r->length;
    out[1] = r->reserved;
    out[2] = r->slot;
    return 0;
}
// The request's table of one group; returns its length (which may exceed `capacity`: call again).
RT_API int chibi_cache_table(void* cache, long long id, int group, int* out, int capacity)
{
    CacheManager* m = static_cast<CacheManager*>(cache);
    const Request* r = m->find(id);
    if (!r)
        return fail(RT_UNKNOWN_REQUEST, "request is not admitted");
    if (group < 0 || group >= m->num_groups())
        return fail(RT_INVALID_CONFIGURATION, "no such group");
    const std::vector<int>& t = r->tables[group];
    for (int i = 0; i < static_cast<int>(t.size()) && i < capacity; ++i)
        out[i] = t[i];
    return static_cast<int>(t.size());
}
RT_API int chibi_cache_reserve(void* cache, long long id, int tokens)
{
    return static_cast<CacheManager*>(cache)->reserve(id, tokens);
}
RT_API int chibi_cache_commit(void* cache, long long id, int new_length)
{
    return static_cast<CacheManager*>(cache)->commit(id, new_length);
}
// A step's requests at once.  what: 0 commit, 1 commit and hold, 2 settle, 3 rollback
// (`lengths` is unused for settle).  Stops at the first failure.
RT_API int chibi_cache_advance(void* cache, int what, int count, const long long* ids, const int* lengths)
{
    CacheManager* m = static_cast<CacheManager*>(cache);
    for (int i = 0; i < count; ++i) {
        int st;
        switch (what) {
        case 0: st = m->commit(ids[i], lengths[i]); break;
        case 1: st = m->commit(ids[i], lengths[i], true); break;
        case 2: st = m->settle(ids[i]); break;
        case 3: st = m->rollback(ids[i], lengths[i]); break;
        default: return fail(RT_INVALID_CONFIGURATION, "chibi_cache_advance: unknown operation");
        }
        if (st < 0)
            return st;
    }
    return 0;
}
RT_API int chibi_cache_release(void* cache, long long id) { return static_cast<CacheManager*>(cache)->release(id); }
RT_API int chibi_cache_free_pages(void* cache, int group)
{
    return static_cast<CacheManager*>(cache)->pool(group).free_count();
}
RT_API int chibi_cache_free_slots(void* cache) { return static_cast<CacheManager*>(cache)->slots().free_count(); }
RT_API int chibi_cache_pending_updates(void* cache, int group)
{
    return static_cast<int>(static_cast<CacheManager*>(cache)->pending_updates(group));
}
// out: (row, index, page) triples; returns their number, or RT_BUFFER_TOO_SMALL (nothing is drained then)
RT_API int chibi_cache_drain(void* cache, int group, int* out, int capacity_triples)
{
    CacheManager* m = static_cast<CacheManager*>(cache);
    if (static_cast<int>(m->pending_updates(group)) > capacity_triples)
        return fail(RT_BUFFER_TOO_SMALL, "more table updates than the caller has room for");
    const std::vector<Update> ups = m->drain(group);
    for (size_t i = 0; i < ups.size(); ++i) {
        out[3 * i] = ups[i].row;
        out[3 * i + 1] = ups[i].index;
        out[3 * i + 2] = ups[i].page;
    }
    return static_cast<int>(ups.size());
}
RT_API int chibi_cache_check(void* cache) { return static_cast<CacheManager*>(cache)->check(); }

// ------------------------------------------------------------------ a step's batch
// Flattens a batch and packs everything the device needs about it into `out` (32-bit
// integers, every segment on a 16-byte boundary):
//   tokens[T] positions[T] seq_of_token[T] q_start[S + 1] ctx_len[S] state_slots[S] logit_rows[R]
//   then, per cache group, 1 + 3 * cap values: the number of table updates and the
//   (row, index, page) triples.
// Entries: request i brings n_tokens[i] tokens (consecutive in `tokens`) and wants the logits at
// n_want[i] places (consecutive in `want`, indices into its own tokens).  Every request gets room
// for its new tokens first (reserve).  With fixed_capacity each group's cap is 2 * S (what a
// captured graph was sized for), else the number of updates; if the updates of a group do not
// fit 2 * S the call falls back to exact capacities and says so in info[5].
// info: T, S, R, words used, largest context length, fixed capacities kept (0 / 1), then the
// offsets of the seven segments and of each group's segment, then each group's cap.
// Checks: no request twice, at least one token each, ids inside the vocabulary, positions
// below the model's limit, wanted places inside the entry.
RT_API int chibi_pack_step(void* cache, int num_entries, const long long* ids, const int* n_tokens,
                           const int* tokens, const int* n_want, const int* want, int vocab_size,
                           int max_positions, int fixed_capacity, int* out, int out_capacity, int* info,
                           int info_capacity)
{
    CacheManager* m = static_cast<CacheManager*>(cache);
    const int G = m->num_groups();
    if (num_entries <= 0)
        return fail(RT_BATCH, "a step needs at least one entry");
    if (info_capacity < 6 + 7 + 2 * G)
        return fail(RT_BUFFER_TOO_SMALL, "info is too small");
    std::unordered_set<long long> seen;
    int T = 0, R = 0;
    for (int i = 0; i < num_entries; ++i) {
        if (!seen.insert(ids[i]).second)
            return fail(RT_BATCH, "entry " + str(i) + ": its request appears twice in one step");
        if (n_tokens[i] <= 0)
            return fail(RT_BATCH, "entry " + str(i) + ": its request brings no tokens");
        if (!m->find(ids[i]))
            return fail(RT_UNKNOWN_REQUEST, "entry " + str(i) + ": its request is not admitted");
        T += n_tokens[i];
        R += n_want[i];
    }
    const int S = num_entries;
    // checks before anything changes
    {
        int tok = 0, w = 0;
        for (int i = 0; i < S; ++i) {
            const Request* r = m->find(ids[i]);
            if (r->length + n_tokens[i] > max_positions)
                return fail(RT_BATCH, "entry " + str(i) + ": its request would reach position "
                                          + str(r->length + n_tokens[i] - 1) + "; the model's limit is "
                                          + str(max_positions - 1));
            for (int j = 0; j < n_tokens[i]; ++j, ++tok)
                if (tokens[tok] < 0 || tokens[tok] >= vocab_size)
                    return fail(RT_BATCH, "entry " + str(i) + ": token id " + str(tokens[tok])
                                              + " is outside the vocabulary of " + str(vocab_size));
            for (int j = 0; j < n_want[i]; ++j, ++w)
                if (want[w] < 0 || want[w] >= n_tokens[i])
                    return fail(RT_BATCH, "entry " + str(i) + ": wanted place " + str(want[w])
                                              + " is outside its " + str(n_tokens[i]) + " tokens");
        }
    }
    for (int i = 0; i < S; ++i) {
        const Request* r = m->find(ids[i]);
        const int st = m->reserve(ids[i], r->length + n_tokens[i]);
        if (st < 0)
            return st;
    }
    {
        // room for the worst case before any update is taken from the manager
        int words = 0;
        const int sizes[7] = { T, T, T, S + 1, S, S, R };
        for (int k = 0; k < 7; ++k)
            words += align4(std::max(sizes[k], 1));
        for (int g = 0; g < G; ++g)
            words += align4(1 + 3 * std::max(2 * S, m->pending_updates(g) > 0 ? (int)m->pending_updates(g) : 0));
        if (words > out_capacity)
            return fail(RT_BUFFER_TOO_SMALL, "the packed batch may need " + str(words) + " words");
    }
    std::vector<std::vector<Update>> ups(G);
    bool fixed = fixed_capacity != 0;
    for (int g = 0; g < G; ++g) {
        ups[g] = m->drain(g);
        if (static_cast<int>(ups[g].size()) > 2 * S)
            fixed = false;
    }
    std::vector<int> cap(G);
    for (int g = 0; g < G; ++g)
        cap[g] = fixed ? 2 * S : static_cast<int>(ups[g].size());
    int offsets[7];
    const int sizes[7] = { T, T, T, S + 1, S, S, R };
    int cursor = 0;
    for (int k = 0; k < 7; ++k) {
        offsets[k] = cursor;
        cursor += align4(std::max(sizes[k], 1));
    }
    std::vector<int> group_offset(G);
    for (int g = 0; g < G; ++g) {
        group_offset[g] = cursor;
        cursor += align4(1 + 3 * cap[g]);
    }
    std::fill(out, out + cursor, 0);
    int* o_tok = out + offsets[0];
    int* o_pos = out + offsets[1];
    int* o_seq = out + offsets[2];
    int* o_qs = out + offsets[3];
    int* o_ctx = out + offsets[4];
    int* o_slot = out + offsets[5];
    int* o_rows = out + offsets[6];
    int t = 0, w = 0, row = 0, max_ctx = 0;
    o_qs[0] = 0;
    for (int i = 0; i < S; ++i) {
        const Request* r = m->find(ids[i]);
        for (int j = 0; j < n_tokens[i]; ++j) {
            o_tok[t + j] = tokens[t + j];
            o_pos[t + j] = r->length + j;
            o_seq[t + j] = i;
        }
        for (int j = 0; j < n_want[i]; ++j, ++w)
            o_rows[row++] = t + want[w];
        t += n_tokens[i];
        o_qs[i + 1] = t;
        o_ctx[i] = r->length + n_tokens[i];
        o_slot[i] = r->slot;
        max_ctx = std::max(max_ctx, o_ctx[i]);
    }
    for (int g = 0; g < G; ++g) {
        int* seg = out + group_offset[g];
        seg[0] = static_cast<int>(ups[g].size());
        for (size_t u = 0; u < ups[g].size(); ++u) {
            seg[1 + 3 * u] = ups[g][u].row;
            seg[2 + 3 * u] = ups[g][u].index;
            seg[3 + 3 * u] = ups[g][u].page;
        }
    }
    info[0] = T;
    info[1] = S;
    info[2] = R;
    info[3] = cursor;
    info[4] = max_ctx;
    info[5] = fixed ? 1 : 0;
    for (int k = 0; k < 7; ++k)
        info[6 + k] = offsets[k];
    for (int g = 0; g < G; ++g) {
        info[13 + g] = group_offset[g];
        info[13 + G + g] = cap[g];
    }
    return 0;
}

// ------------------------------------------------------------------ scheduler
// Admits requests, cuts prompts into portions under a token budget, decodes,
// finishes.  Kept from the reference (src/scheduler.cc, src/seq.cc): a sequence is
// waiting (prompt not fully processed), running (one token per step) or finished;
// after the last portion of the prompt the sampled token is appended unprocessed, and
// every decode step processes it and appends the next (src/seq.cc:138-160,
// src/scheduler.cc:393-398); admission is three-way (src/scheduler.cc:162-235); the page
// budget is the worst case of every live request, so pages cannot run out in the middle
// of a request (src/scheduler.cc:13-22); a portion is min(what is left, quantum, what
// the step's budget has left), the quantum being prefill_chunk_tokens while requests
// compete and the whole budget otherwise (src/scheduler.cc:259-275); a prompt that was
// not finished goes to the back of the waiting queue (src/scheduler.cc:376-383); stop:
// EOS first, then length (src/seq.cc:287-303).  Changed: every step takes one token of
// every running sequence first and fills what is left of the budget with prompt
// portions, in one mixed batch.
//
// The scheduler reserves pages itself (it shares the cache manager) but neither admits
// requests to the cache nor releases them: its caller does, when told.
namespace {

enum : int {
    SC_BATCH_IN_FLIGHT = -20,
    SC_DUPLICATE_SEQUENCE = -21,
    SC_INVALID_SEQUENCE_STATE = -22,
    SC_NO_RUNNABLE_SEQUENCES = -23,
    SC_CACHE_CAPACITY_EXHAUSTED = -24,
    SC_BLOCK_MANAGER_FAILURE = -25,
    SC_NO_BATCH_IN_FLIGHT = -26,
    SC_BATCH_ID_MISMATCH = -27,
    SC_RESULT_COUNT_MISMATCH = -28,
    SC_UNKNOWN_SEQUENCE = -29,
    SC_SEQUENCE_NOT_FINISHED = -30,
    SC_INVALID_CONFIGURATION = -31,
};

enum : int { ST_WAITING = 0, ST_RUNNING = 1, ST_FINISHED = 2 };
enum : int { FR_NONE = 0, FR_EOS = 1, FR_LEN_LIMIT = 2, FR_CANCELLED = 3 };
enum : int { AD_ADMITTED = 0, AD_DEFERRED = 1, AD_TOO_LARGE = 2 };

struct Seq {
    std::vector<int> tokens;
    int prompt_len = 0, processed = 0, scheduled = 0, status = ST_WAITING, reason = FR_NONE;
    int max_new_tokens = 0;
    bool ignore_eos = false;
    int schedulable() const { return static_cast<int>(tokens.size()) - processed - scheduled; }
    int completion_len() const { return static_cast<int>(tokens.size()) - prompt_len; }
};

struct Item {
    long long id;
    int first, count, sample;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int max_sequences, int max_batch_tokens, int prefill_chunk_tokens, int eos)
        : cache_(cache), max_sequences_(max_sequences), max_batch_tokens_(max_batch_tokens),
          prefill_chunk_tokens_(prefill_chunk_tokens), eos_(eos)
    {
    }
    bool active() const { return active_; }
    int active_id() const { return active_id_; }
    const std::vector<Item>& active_items() const { return items_; }
    const std::deque<long long>& queue(int which) const { return which ? running_ : waiting_; }
    Seq* find(long long id)
    {
        auto it = seqs_.find(id);
        return it == seqs_.end() ? nullptr : &it->second;
    }
    static int budget_tokens(int prompt_len, int max_new_tokens) { return prompt_len + max_new_tokens - 1; }
    bool fits_cache(int prompt_len, int max_new_tokens) const
    {
        for (int g = 0; g < cache_->num_groups(); ++g)
            if (pages_for(budget_tokens(prompt_len, max_new_tokens), cache_->group(g).page_size)
                > cache_->group(g).num_pages)
                return false;
        return true;
    }
    int admission(int prompt_len, int max_new_tokens) const
    {
        if (active_)
            return fail(SC_BATCH_IN_FLIGHT, "a batch is in flight");
        if (!fits_cache(prompt_len, max_new_tokens))
            return AD_TOO_LARGE;
        if (static_cast<int>(waiting_.size() + running_.size()) >= max_sequences_)
            return AD_DEFERRED;
        for (int g = 0; g < cache_->num_groups(); ++g) {
            const int page_size = cache_->group(g).page_size;
            int available = cache_->group(g).num_pages;
            for (const auto* q : { &waiting_, &running_ })
                for (long long id : *q) {
                    const Seq& s = seqs_.at(id);
                    available -= pages_for(budget_tokens(s.prompt_len, s.max_new_tokens), page_size);
                }
            if (pages_for(budget_tokens(prompt_len, max_new_tokens), page_size) > available)
                return AD_DEFERRED;
        }
        return AD_ADMITTED;
    }
    int add(long long id, const int* prompt, int prompt_len, int max_new_tokens, bool ignore_eos)
    {
        if (active_)
            return fail(SC_BATCH_IN_FLIGHT, "a batch is in flight");
        if (seqs_.count(id))
            return fail(SC_DUPLICATE_SEQUENCE, "the sequence is already known");
        if (prompt_len <= 0 || max_new_tokens <= 0)
            return fail(SC_INVALID_SEQUENCE_STATE, "a sequence needs a prompt and a positive token limit");
        Seq s;
        s.tokens.assign(prompt, prompt + prompt_len);
        s.prompt_len = prompt_len;
        s.max_new_tokens = max_new_tokens;
        s.ignore_eos = ignore_eos;
        seqs_.emplace(id, std::move(s));
        waiting_.push_back(id);
        return 0;
    }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int schedule()
    {
        if (active_)
            return fail(SC_BATCH_IN_FLIGHT, "a batch is in flight");
        if (!has_work())
            return fail(SC_NO_RUNNABLE_SEQUENCES, "nothing to run");
        items_.clear();
        int used = 0;
        auto full = [&] { return static_cast<int>(items_.size()) >= max_sequences_ || used >= max_batch_tokens_; };
        auto take = [&](long long id, Seq& s, int count) -> int {
            const int st = cache_->reserve(id, s.processed + count);
            if (st < 0)
                return fail(st == RT_CAPACITY_EXHAUSTED ? SC_CACHE_CAPACITY_EXHAUSTED : SC_BLOCK_MANAGER_FAILURE,
                            g_error);
            items_.push_back({ id, s.processed, count, count == s.schedulable() ? 1 : 0 });
            s.scheduled = count;
            used += count;
            return 0;
        };
        int status = 0;
        for (long long id : running_) {
            if (full())
                break;
            Seq& s = seqs_.at(id);
            if (s.schedulable() != 1) {
                status = fail(SC_INVALID_SEQUENCE_STATE, "a running sequence has " + str(s.schedulable())
                                                             + " tokens to run");
                break;
            }
            if ((status = take(id, s, 1)) < 0)
                break;
        }
        if (status == 0) {
            const bool contended = waiting_.size() > 1 || !running_.empty();
            const int quantum = contended ? prefill_chunk_tokens_ : max_batch_tokens_;
            for (long long id : waiting_) {
                if (full())
                    break;
                Seq& s = seqs_.at(id);
                const int available = s.schedulable();
                if (available <= 0) {
                    status = fail(SC_INVALID_SEQUENCE_STATE, "a waiting sequence has nothing to run");
                    break;
                }
                const int count = std::min({ available, quantum, max_batch_tokens_ - used });
                if ((status = take(id, s, count)) < 0)
                    break;
            }
        }
        if (status == 0 && items_.empty())
            status = fail(SC_NO_RUNNABLE_SEQUENCES, "nothing to run");
        if (status < 0) {
            const std::string keep = g_error;
            rollback();
            g_error = keep;
            return status;
        }
        active_ = true;
        active_id_ = next_batch_++;
        return static_cast<int>(items_.size());
    }
    // updates: (id, token, finish reason) per sampling item, in the order of the items
    int complete(int batch_id, const int* sampled, int n_sampled, std::vector<long long>* updates)
    {
        if (!active_)
            return fail(SC_NO_BATCH_IN_FLIGHT, "no batch is in flight");
        if (batch_id != active_id_)
            return fail(SC_BATCH_ID_MISMATCH, "another batch is in flight");
        int samples = 0;
        for (const Item& it : items_)
            samples += it.sample;
        if (n_sampled != samples)
            return fail(SC_RESULT_COUNT_MISMATCH, str(n_sampled) + " samples for " + str(samples) + " sampling items");
        int k = 0;
        for (const Item& it : items_) {
            Seq& s = seqs_.at(it.id);
            s.processed += s.scheduled;
            s.scheduled = 0;
            const bool was_waiting = s.status == ST_WAITING;
            std::deque<long long>& q = was_waiting ? waiting_ : running_;
            q.erase(std::find(q.begin(), q.end(), it.id));
            if (!it.sample) {
                waiting_.push_back(it.id);
                continue;
            }
            if (was_waiting)
                s.status = ST_RUNNING;
            s.tokens.push_back(sampled[k++]);
            int reason = FR_NONE;
            if (!s.ignore_eos && eos_ >= 0 && s.tokens.back() == eos_)
                reason = FR_EOS;
            else if (s.completion_len() >= s.max_new_tokens)
                reason = FR_LEN_LIMIT;
            if (reason != FR_NONE) {
                s.status = ST_FINISHED;
                s.reason = reason;
            } else {
                running_.push_back(it.id);
            }
            updates->push_back(it.id);
            updates->push_back(s.tokens.back());
            updates->push_back(reason);
        }
        active_ = false;
        items_.clear();
        return static_cast<int>(updates->size() / 3);
    }
    int abort(int batch_id)
    {
        if (!active_)
            return fail(SC_NO_BATCH_IN_FLIGHT, "no batch is in flight");
        if (batch_id != active_id_)
            return fail(SC_BATCH_ID_MISMATCH, "another batch is in flight");
        rollback();
        return 0;
    }
    // 1: the sequence was live and is now finished (its caller releases its cache); 0: it had finished
    int cancel(long long id)
    {
        if (active_)
            return fail(SC_BATCH_IN_FLIGHT, "a batch is in flight");
        Seq* s = find(id);
        if (!s)
            return fail(SC_UNKNOWN_SEQUENCE, "no such sequence");
        if (s->status == ST_FINISHED)
            return 0;
        for (auto* q : { &waiting_, &running_ }) {
            auto it = std::find(q->begin(), q->end(), id);
            if (it != q->end())
                q->erase(it);
        }
        s->status = ST_FINISHED;
        s->reason = FR_CANCELLED;
        s->scheduled = 0;
        return 1;
    }
    int remove(long long id)
    {
        Seq* s = find(id);
        if (!s)
            return fail(SC_UNKNOWN_SEQUENCE, "no such sequence");
        if (s->status != ST_FINISHED)
            return fail(SC_SEQUENCE_NOT_FINISHED, "the sequence has not finished");
        seqs_.erase(id);
        return 0;
    }
    int check() const
    {
        std::unordered_set<long long> live;
        for (const auto* q : { &waiting_, &running_ })
            for (long long id : *q)
                if (!live.insert(id).second)
                    return fail(RT_INVARIANT, "a sequence is queued twice");
        for (const auto& kv : seqs_) {
            const Seq& s = kv.second;
            if (s.processed < 0 || s.scheduled < 0 || s.processed + s.scheduled > static_cast<int>(s.tokens.size()))
                return fail(RT_INVARIANT, "a sequence's counters are out of order");
            const bool in_waiting = std::find(waiting_.begin(), waiting_.end(), kv.first) != waiting_.end();
            const bool in_running = std::find(running_.begin(), running_.end(), kv.first) != running_.end();
            if (s.status == ST_WAITING && !in_waiting)
                return fail(RT_INVARIANT, "a waiting sequence is not in the waiting queue");
            if (s.status == ST_RUNNING && (!in_running || s.schedulable() + s.scheduled != 1))
                return fail(RT_INVARIANT, "a running sequence is not in the running queue with one token to run");
            if (s.status == ST_FINISHED && (in_waiting || in_running))
                return fail(RT_INVARIANT, "a finished sequence is still queued");
        }
        return 0;
    }

private:
    void rollback()
    {
        for (const Item& it : items_)
            seqs_.at(it.id).scheduled = 0;
        items_.clear();
        active_ = false;
    }
    CacheManager* cache_;
    int max_sequences_, max_batch_tokens_, prefill_chunk_tokens_, eos_;
    std::unordered_map<long long, Seq> seqs_;
    std::deque<long long> waiting_, running_;
    bool active_ = false;
    int active_id_ = -1, next_batch_ = 0;
    std::vector<Item> items_;
};

} // namespace

// eos < 0: the model has no end-of-sequence token
RT_API void* chibi_sched_new(void* cache, int max_sequences, int max_batch_tokens, int prefill_chunk_tokens, int eos)
{
    if (!cache || max_sequences <= 0 || max_batch_tokens <= 0 || prefill_chunk_tokens <= 0) {
        fail(SC_INVALID_CONFIGURATION, "max_sequences, max_batch_tokens and prefill_chunk_tokens must be positive");
        return nullptr;
    }
    return new Scheduler(static_cast<CacheManager*>(cache), max_sequences, max_batch_tokens, prefill_chunk_tokens, eos);
}
RT_API void chibi_sched_delete(void* s) { delete static_cast<Scheduler*>(s); }
RT_API int chibi_sched_fits_cache(void* s, int prompt_len, int max_new_tokens)
{
    return static_cast<Scheduler*>(s)->fits_cache(prompt_len, max_new_tokens) ? 1 : 0;
}
// 0 admitted, 1 deferred, 2 too large
RT_API int chibi_sched_admission(void* s, int prompt_len, int max_new_tokens)
{
    return static_cast<Scheduler*>(s)->admission(prompt_len, max_new_tokens);
}
RT_API int chibi_sched_add(void* s, long long id, const int* prompt, int prompt_len, int max_new_tokens,
                           int ignore_eos)
{
    return static_cast<Scheduler*>(s)->add(id, prompt, prompt_len, max_new_tokens, ignore_eos != 0);
}
RT_API int chibi_sched_has_work(void* s) { return static_cast<Scheduler*>(s)->has_work() ? 1 : 0; }
RT_API int chibi_sched_active(void* s) { return static_cast<Scheduler*>(s)->active() ? 1 : 0; }
// items: (id, first, count, sample) per item; returns their number
RT_API int chibi_sched_schedule(void* s, long long* items, int capacity_items, int* batch_id)
{
    Scheduler* sc = static_cast<Scheduler*>(s);
    const int n = sc->schedule();
    if (n < 0)
        return n;
    if (n > capacity_items) {
        sc->abort(sc->active_id());
        return fail(RT_BUFFER_TOO_SMALL, "more items than the caller has room for");
    }
    const std::vector<Item>& its = sc->active_items();
    for (int i = 0; i < n; ++i) {
        items[4 * i] = its[i].id;
        items[4 * i + 1] = its[i].first;
        items[4 * i + 2] = its[i].count;
        items[4 * i + 3] = its[i].sample;
    }
    *batch_id = sc->active_id();
    return n;
}
// updates: (id, token, finish reason: 0 none, 1 eos, 2 len_limit) per sampling item
RT_API int chibi_sched_complete(void* s, int batch_id, const int* sampled, int n_sampled, long long* updates,
                                int capacity_updates)
{
    std::vector<long long> out;
    const int n = static_cast<Scheduler*>(s)->complete(batch_id, sampled, n_sampled, &out);
    if (n < 0)
        return n;
    if (n > capacity_updates)
        return fail(RT_BUFFER_TOO_SMALL, "more updates than the caller has room for");
    std::copy(out.begin(), out.end(), updates);
    return n;
}
RT_API int chibi_sched_abort(void* s, int batch_id) { return static_cast<Scheduler*>(s)->abort(batch_id); }
RT_API int chibi_sched_cancel(void* s, long long id) { return static_cast<Scheduler*>(s)->cancel(id); }
RT_API int chibi_sched_remove(void* s, long long id) { return static_cast<Scheduler*>(s)->remove(id); }
// out: processed, scheduled, status (0 waiting, 1 running, 2 finished), finish reason, tokens, prompt tokens
RT_API int chibi_sched_info(void* s, long long id, int* out)
{
    const Seq* q = static_cast<Scheduler*>(s)->find(id);
    if (!q)
        return fail(SC_UNKNOWN_SEQUENCE, "no such sequence");
    out[0] = q->processed;
    out[1] = q->scheduled;
    out[2] = q->status;
    out[3] = q->reason;
    out[4] = static_cast<int>(q->tokens.size());
    out[5] = q->prompt_len;
    return 0;
}
// tokens [first, first + count) of a sequence
RT_API int chibi_sched_tokens(void* s, long long id, int first, int count, int* out)
{
    const Seq* q = static_cast<Scheduler*>(s)->find(id);
    if (!q)
        return fail(SC_UNKNOWN_SEQUENCE, "no such sequence");
    if (first < 0 || count < 0 || first + count > static_cast<int>(q->tokens.size()))
        return fail(SC_INVALID_SEQUENCE_STATE, "tokens outside the sequence");
    std::copy(q->tokens.begin() + first, q->tokens.begin() + first + count, out);
    return count;
}
// which: 0 waiting, 1 running; returns the queue's length (which may exceed `capacity`)
RT_API int chibi_sched_queue(void* s, int which, long long* out, int capacity)
{
    const std::deque<long long>& q = static_cast<Scheduler*>(s)->queue(which);
    int i = 0;
    for (long long id : q) {
        if (i < capacity)
            out[i] = id;
        ++i;
    }
    return i;
}
RT_API int chibi_sched_check(void* s) { return static_cast<Scheduler*>(s)->check(); }
