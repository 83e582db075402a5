// Host side of the paged cache: page pools, block tables, request slots, and the packing of a
// step's batch descriptor.  Plain C interface (loaded with ctypes); no GPU call in this file.
//
// The reference's Llama 4 cache is a ring buffer per layer with one shared write cursor
// (llama4/llama4_jax/model.py:595-640) that never gives memory back.  Its paged cache (llama3 only,
// llama3/llama3_jax/model.py:457-553) keeps a free-page bitmap and block tables on the device and has
// no check for running out of pages.  Here pages are handed out and taken back on the host:
//
//  * A *group* is a set of layers with the same need: all keys (kind 0), the keys of the current
//    chunk of `size` positions (kind 1), or the last `size` keys (kind 2).  Each group has its own
//    pool of pages and its own block table; a page id means the same slot in every layer of the group.
//  * A *slot* is a live request: its committed length, its reserved length and one block-table row
//    per group (logical page index = position / page_size -> page id, -1 where nothing is held).
//    The slot id also indexes the fixed-size per-request state of layers that keep one.
//  * reserve(slot, new_len) takes pages for positions [reserved, new_len) in every group, or takes
//    nothing and reports failure.  commit(slot, new_len) records that the step ran and gives back the
//    pages that no later query of the request can read.  release(slot) gives back everything.
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

enum Kind { ALL = 0, CHUNK = 1, WINDOW = 2 };

struct Group {
  int kind = ALL;
  int size = 0;
  int num_pages = 0;
  std::vector<int32_t> free_stack;      // LIFO: a page given back is the next one handed out
  std::vector<uint8_t> held;            // 1 while a block table holds the page
  std::vector<int32_t> table;           // [max_slots][max_pages_per_req]
  std::vector<int32_t> first_held;      // per slot: lowest logical page that may still be held
};

struct Slot {
  bool live = false;
  int64_t committed = 0;
  int64_t reserved = 0;
};

struct Manager {
  int page_size, max_slots, max_pages_per_req;
  std::vector<Group> groups;
  std::vector<Slot> slots;
  std::vector<int32_t> free_slots;  // LIFO
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// First position that a query at position p (and every later one) can still read.
inline int64_t first_needed(const Group& g, int64_t p) {
  if (g.kind == CHUNK) return (p / g.size) * (int64_t)g.size;
  if (g.kind == WINDOW) return p - g.size + 1 > 0 ? p - g.size + 1 : 0;
  return 0;
}

}  // namespace

#define API extern "C" __attribute__((visibility("default")))

API void* cm_create(int page_size, int max_slots, int max_pages_per_req) {
  if (page_size <= 0 || max_slots <= 0 || max_pages_per_req <= 0) return nullptr;
  Manager* m = new Manager();
  m->page_size = page_size;
  m->max_slots = max_slots;
  m->max_pages_per_req = max_pages_per_req;
  m->slots.resize(max_slots);
  for (int s = max_slots - 1; s >= 0; --s) m->free_slots.push_back(s);
  return m;
}

API void cm_destroy(void* h) { delete static_cast<Manager*>(h); }

API int cm_add_group(void* h, int kind, int size, int num_pages) {
  Manager* m = static_cast<Manager*>(h);
  if (kind < ALL || kind > WINDOW || num_pages <= 0 || (kind != ALL && size <= 0)) return -1;
  Group g;
  g.kind = kind;
  g.size = size;
  g.num_pages = num_pages;
  g.held.assign(num_pages, 0);
  for (int p = num_pages - 1; p >= 0; --p) g.free_stack.push_back(p);
  g.table.assign((size_t)m->max_slots * m->max_pages_per_req, -1);
  g.first_held.assign(m->max_slots, 0);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

API int cm_num_groups(void* h) { return (int)static_cast<Manager*>(h)->groups.size(); }
API int cm_free_pages(void* h, int g) { return (int)static_cast<Manager*>(h)->groups[g].free_stack.size(); }
API int cm_num_pages(void* h, int g) { return static_cast<Manager*>(h)->groups[g].num_pages; }
API int cm_free_slot_count(void* h) { return (int)static_cast<Manager*>(h)->free_slots.size(); }
API int32_t* cm_table(void* h, int g) { return static_cast<Manager*>(h)->groups[g].table.data(); }

API int cm_alloc_slot(void* h) {
  Manager* m = static_cast<Manager*>(h);
  if (m->free_slots.empty()) return -1;
  const int s = m->free_slots.back();
  m->free_slots.pop_back();
  m->slots[s] = Slot();
  m->slots[s].live = true;
  for (Group& g : m->groups) g.first_held[s] = 0;
  return s;
}

API long long cm_committed(void* h, int s) {
  Manager* m = static_cast<Manager*>(h);
  return (s < 0 || s >= m->max_slots || !m->slots[s].live) ? -1 : m->slots[s].committed;
}

API long long cm_reserved(void* h, int s) {
  Manager* m = static_cast<Manager*>(h);
  return (s < 0 || s >= m->max_slots || !m->slots[s].live) ? -1 : m->slots[s].reserved;
}

// Pages that every group lacks for the request to reach new_len (0 if none); -1 for a bad slot,
// -2 if new_len does not fit a block-table row.
API int cm_pages_needed(void* h, int s, long long new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
  if (ceil_div(new_len, m->page_size) > m->max_pages_per_req) return -2;
  const Slot& sl = m->slots[s];
  if (new_len <= sl.reserved) return 0;
  return (int)(ceil_div(new_len, m->page_size) - ceil_div(sl.reserved, m->page_size));
}

// 0 = reserved; 1 = not enough free pages in some group (nothing taken); negative = misuse.
API int cm_reserve(void* h, int s, long long new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
  Slot& sl = m->slots[s];
  if (new_len <= sl.reserved) return 0;
  const int64_t lo = ceil_div(sl.reserved, m->page_size), hi = ceil_div(new_len, m->page_size);
  if (hi > m->max_pages_per_req) return -2;
  for (const Group& g : m->groups)
    if ((int64_t)g.free_stack.size() < hi - lo) return 1;
  for (Group& g : m->groups) {
    int32_t* row = g.table.data() + (size_t)s * m->max_pages_per_req;
    for (int64_t i = lo; i < hi; ++i) {
      const int32_t p = g.free_stack.back();
      g.free_stack.pop_back();
      g.held[p] = 1;
      row[i] = p;
    }
  }
  sl.reserved = new_len;
  return 0;
}

// The step that filled positions [committed, new_len) has been launched.  Gives back, per group, the
// pages wholly before the first position that the request's next query can read.  Returns the
// number of pages given back, or a negative code for misuse.
API int cm_commit(void* h, int s, long long new_len) {
  Manager* m = static_cast<Manager*>(h);
  if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
  Slot& sl = m->slots[s];
  if (new_len < sl.committed || new_len > sl.reserved) return -3;
  sl.committed = new_len;
  int freed = 0;
  for (Group& g : m->groups) {
    if (g.kind == ALL) continue;
    const int64_t dead_pages = first_needed(g, new_len) / m->page_size;  // pages [0, dead_pages) are dead
    int32_t* row = g.table.data() + (size_t)s * m->max_pages_per_req;
    for (int64_t i = g.first_held[s]; i < dead_pages; ++i) {
      const int32_t p = row[i];
      if (p >= 0) {
        g.held[p] = 0;
        g.free_stack.push_back(p);
        row[i] = -1;
        ++freed;
      }
    }
    if (dead_pages > g.first_held[s]) g.first_held[s] = (int32_t)dead_pages;
  }
  return freed;
}

// Gives back every page of the request and its slot.  Returns pages given back; -1 if the slot is
// not live (a second release is refused, not repeated).
API int cm_release(void* h, int s) {
  Manager* m = static_cast<Manager*>(h);
  if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
  Slot& sl = m->slots[s];
  const int64_t hi = ceil_div(sl.reserved, m->page_size);
  int freed = 0;
  for (Group& g : m->groups) {
    int32_t* row = g.table.data() + (size_t)s * m->max_pages_per_req;
    for (int64_t i = g.first_held[s]; i < hi; ++i) {
      const int32_t p = row[i];
      if (p >= 0) {
        g.held[p] = 0;
        g.free_stack.push_back(p);
        row[i] = -1;
        ++freed;
      }
    }
    g.first_held[s] = 0;
  }
  sl = Slot();
  m->free_slots.push_back(s);
  return freed;
}

API int cm_pages_held(void* h, int s, int g) {
  Manager* m = static_cast<Manager*>(h);
  if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
  const int32_t* row = m->groups[g].table.data() + (size_t)s * m->max_pages_per_req;
  int n = 0;
  for (int i = 0; i < m->max_pages_per_req; ++i) n += row[i] >= 0;
  return n;
}

// Invariants: every page is either on the free stack once or in exactly one block-table entry of a
// live slot; dead slots hold nothing.  0 = sound; otherwise a code naming the first fault found.
API int cm_check(void* h) {
  Manager* m = static_cast<Manager*>(h);
  for (const Group& g : m->groups) {
    std::vector<int> seen(g.num_pages, 0);
    for (int32_t p : g.free_stack) {
      if (p < 0 || p >= g.num_pages) return 1;
      if (seen[p]++) return 2;      // on the free stack twice
      if (g.held[p]) return 3;      // free and held
    }
    for (int s = 0; s < m->max_slots; ++s) {
      const int32_t* row = g.table.data() + (size_t)s * m->max_pages_per_req;
      for (int i = 0; i < m->max_pages_per_req; ++i) {
        const int32_t p = row[i];
        if (p < 0) continue;
        if (!m->slots[s].live) return 4;  // a dead slot holds a page
        if (p >= g.num_pages) return 1;
        if (seen[p]++) return 5;          // held twice, or held and free
        if (!g.held[p]) return 6;
      }
    }
    for (int p = 0; p < g.num_pages; ++p)
      if (!seen[p]) return 7;  // lost: neither free nor held
  }
  std::vector<int> slot_seen(m->max_slots, 0);
  for (int32_t s : m->free_slots) {
    if (s < 0 || s >= m->max_slots || slot_seen[s]++ || m->slots[s].live) return 8;
  }
  for (int s = 0; s < m->max_slots; ++s)
    if (!m->slots[s].live && !slot_seen[s]) return 9;
  return 0;
}

// Packs the descriptor of one step into `out` (int32, caller-sized):
//   token_ids[N] positions[N] req_of_token[N] cu_q[R+1] q_start[R] kv_len[R] slot_ids[R] logit_rows[M]
//   then per group a block table [R][width].
// Request r brings n_tokens[r] tokens starting at its committed length; want_* is a CSR list of the
// places (within the request's tokens) whose logits are asked for.  Returns the number of int32
// written, or a negative code: -1 bad slot, -2 positions not reserved, -3 a wanted place out of range,
// -4 width too small.
API long long cm_pack_step(void* h, int R, const int32_t* slot_ids, const int32_t* n_tokens, const int32_t* tokens,
                           const int32_t* want_offsets, const int32_t* want, int width, int N_pad, int R_pad, int M_pad,
                           int32_t* out) {
  Manager* m = static_cast<Manager*>(h);
  int64_t N = 0;
  for (int r = 0; r < R; ++r) N += n_tokens[r];
  const int64_t M = want_offsets[R];
  if (N > N_pad || R > R_pad || M > M_pad) return -5;
  int32_t* token_ids = out;
  int32_t* positions = token_ids + N_pad;
  int32_t* req_of_token = positions + N_pad;
  int32_t* cu_q = req_of_token + N_pad;
  int32_t* q_start = cu_q + (R_pad + 1);
  int32_t* kv_len = q_start + R_pad;
  int32_t* slots_out = kv_len + R_pad;
  int32_t* logit_rows = slots_out + R_pad;
  int32_t* tables = logit_rows + M_pad;
  const size_t G = m->groups.size();
  int64_t at = 0;
  for (int r = 0; r < R; ++r) {
    const int s = slot_ids[r];
    if (s < 0 || s >= m->max_slots || !m->slots[s].live) return -1;
    const Slot& sl = m->slots[s];
    const int64_t start = sl.committed, n = n_tokens[r];
    if (start + n > sl.reserved) return -2;
    if (ceil_div(start + n, m->page_size) > width) return -4;
    cu_q[r] = (int32_t)at;
    q_start[r] = (int32_t)start;
    kv_len[r] = (int32_t)(start + n);
    slots_out[r] = s;
    for (int64_t i = 0; i < n; ++i) {
      token_ids[at + i] = tokens[at + i];
      positions[at + i] = (int32_t)(start + i);
      req_of_token[at + i] = r;
    }
    for (int j = want_offsets[r]; j < want_offsets[r + 1]; ++j) {
      if (want[j] < 0 || want[j] >= n) return -3;
      logit_rows[j] = (int32_t)(at + want[j]);
    }
    for (size_t g = 0; g < G; ++g) {
      const int32_t* row = m->groups[g].table.data() + (size_t)s * m->max_pages_per_req;
      int32_t* dst = tables + (g * R_pad + r) * (size_t)width;
      const int copy = width < m->max_pages_per_req ? width : m->max_pages_per_req;
      std::memcpy(dst, row, sizeof(int32_t) * copy);
      for (int i = copy; i < width; ++i) dst[i] = -1;
    }
    at += n;
  }
  cu_q[R] = (int32_t)at;
  // padding: rows beyond the live ones repeat harmless values (position 0 of request 0 is never
  // written because padded tokens are not run; tables of padded requests hold -1)
  for (int64_t i = N; i < N_pad; ++i) { token_ids[i] = 0; positions[i] = 0; req_of_token[i] = 0; }
  for (int r = R; r < R_pad; ++r) {
    cu_q[r + 1] = (int32_t)at; q_start[r] = 0; kv_len[r] = 0; slots_out[r] = -1;
    for (size_t g = 0; g < G; ++g) {
      int32_t* dst = tables + (g * R_pad + r) * (size_t)width;
      for (int i = 0; i < width; ++i) dst[i] = -1;
    }
  }
  for (int64_t j = M; j < M_pad; ++j) logit_rows[j] = 0;
  return (long long)(3 * (int64_t)N_pad + (R_pad + 1) + 3 * (int64_t)R_pad + M_pad + (int64_t)G * R_pad * width);
}
