// Host-side runtime of the step function, in C++: the cache's bookkeeping (slots, pages per group of layers,
// lengths, windows) and the plan of one step (checks before any launch, page reservation, the packed int32
// step buffer that every kernel reads).  No CUDA here; Python holds the handles and raises the typed errors.
//
// The reference keeps these on the native side of its facade too: the per-sequence state and its append-only
// length (crates/model/src/qwen35/state.rs:30-57, crates/model/src/cache.rs:10-37 for windows), the limits
// checked before a forward pass (crates/gpu/src/qwen35.rs:1212-1222, crates/model/src/qwen35/cpu.rs:119-125).
//
// A *slot* is one live sequence's entry.  A *page* holds LLMX_PAGE consecutive positions of one sequence for
// every layer of one group.  Position p lives in logical page p / LLMX_PAGE; a slot's page list maps logical to
// physical pages (-1 where a window group has given a page back).  Lengths only grow.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define LLMX_API extern "C" __attribute__((visibility("default")))
#define LLMX_PAGE 64

namespace {

enum Code { OK = 0, MISUSE = 1, OVERFLOW_SEQ = 2, EXHAUSTED = 3, BAD_VALUE = 4, OVERFLOW_STEP = 5, TOO_SMALL = 6 };

thread_local std::string g_error;
thread_local long long g_info[2];      // numbers that go with the error (tokens, limit)

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

inline long long pages_for(long long n) { return (n + LLMX_PAGE - 1) / LLMX_PAGE; }

struct Pool {
  int n_pages = 0;
  std::vector<int> free_list;     // back() is handed out next; low ids first
  std::vector<char> held;
  explicit Pool(int n) : n_pages(n), held(n, 0) {
    for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
  }
  int n_free() const { return (int)free_list.size(); }
  int take() {
    const int p = free_list.back();
    free_list.pop_back();
    held[p] = 1;
    return p;
  }
  int give_back(int p) {
    if (p < 0 || p >= n_pages || !held[p]) return fail(MISUSE, "page %d is given back but is not held", p);
    held[p] = 0;
    free_list.push_back(p);
    return OK;
  }
};

struct Slot {
  long long length = 0, reserved = 0, generation = 0;
  bool live = false;
  std::vector<std::vector<int>> pages;      // per group: logical page -> physical page or -1
};

struct Allocator {
  int n_slots, n_pages;
  long long max_seq_len;
  std::vector<int> windows;                  // per group; <= 0: every earlier key
  std::vector<Pool> pools;
  std::vector<Slot> slots;
  std::vector<int> free_slots;               // back() is handed out next

  Allocator(int ns, int np, const int* w, int ng, long long max_len)
      : n_slots(ns), n_pages(np), max_seq_len(max_len), windows(w, w + ng), slots(ns) {
    for (int g = 0; g < ng; ++g) pools.emplace_back(np);
    for (int s = ns - 1; s >= 0; --s) free_slots.push_back(s);
  }

  Slot* live(int slot) {
    if (slot < 0 || slot >= n_slots) {
      fail(MISUSE, "slot %d does not exist (there are %d)", slot, n_slots);
      return nullptr;
    }
    if (!slots[slot].live) {
      fail(MISUSE, "slot %d is not held by a live sequence (freed twice, or used after being freed)", slot);
      return nullptr;
    }
    return &slots[slot];
  }

  int acquire() {
    if (free_slots.empty()) return -fail(EXHAUSTED, "all %d cache slots are held by live sequences", n_slots);
    const int s = free_slots.back();
    free_slots.pop_back();
    Slot& st = slots[s];
    st.length = st.reserved = 0;
    st.pages.assign(pools.size(), {});
    st.live = true;
    ++st.generation;
    return s;
  }

  int release(int slot) {
    Slot* st = live(slot);
    if (!st) return MISUSE;
    for (size_t g = 0; g < pools.size(); ++g)
      for (int p : st->pages[g])
        if (p >= 0 && pools[g].give_back(p)) return MISUSE;
    st->pages.assign(pools.size(), {});
    st->length = st->reserved = 0;
    st->live = false;
    free_slots.push_back(slot);
    return OK;
  }

  // Makes sure positions length .. length + n_new - 1 have pages in every group; nothing changes if they do not fit.
  int reserve(int slot, long long n_new) {
    Slot* st = live(slot);
    if (!st) return MISUSE;
    const long long new_len = st->length + n_new;
    if (new_len > max_seq_len) {
      g_info[0] = new_len, g_info[1] = max_seq_len;
      return fail(OVERFLOW_SEQ, "%lld tokens do not fit the longest sequence the cache allows of %lld", new_len, max_seq_len);
    }
    const long long want = pages_for(new_len);
    for (size_t g = 0; g < pools.size(); ++g) {
      const long long need = want - (long long)st->pages[g].size();
      if (need > pools[g].n_free())
        return fail(EXHAUSTED, "slot %d needs %lld more cache pages for %lld positions, %d of %d are free", slot, need,
                    new_len, pools[g].n_free(), pools[g].n_pages);
    }
    for (size_t g = 0; g < pools.size(); ++g)
      while ((long long)st->pages[g].size() < want) st->pages[g].push_back(pools[g].take());
    st->reserved = std::max(st->reserved, new_len);
    return OK;
  }

  // Takes back a reservation that no step will use.
  int unreserve(int slot) {
    Slot* st = live(slot);
    if (!st) return MISUSE;
    const size_t keep = (size_t)pages_for(st->length);
    for (size_t g = 0; g < pools.size(); ++g) {
      auto& pages = st->pages[g];
      for (size_t i = keep; i < pages.size(); ++i)
        if (pages[i] >= 0 && pools[g].give_back(pages[i])) return MISUSE;
      if (pages.size() > keep) pages.resize(keep);
    }
    st->reserved = st->length;
    return OK;
  }

  // The step wrote n_new positions: the length grows, and groups with a window give back the pages that no
  // later query can see (the next query sits at `length` and sees keys from length - (window - 1) on).
  int commit(int slot, long long n_new) {
    Slot* st = live(slot);
    if (!st) return MISUSE;
    if (st->length + n_new > st->reserved)
      return fail(MISUSE, "slot %d: %lld positions are committed but only %lld were reserved", slot, n_new,
                  st->reserved - st->length);
    st->length += n_new;
    for (size_t g = 0; g < pools.size(); ++g) {
      if (windows[g] <= 0) continue;
      const long long first_visible = std::max(0LL, st->length - (windows[g] - 1));
      const long long dead = std::min<long long>(first_visible / LLMX_PAGE, (long long)st->pages[g].size());
      for (long long i = 0; i < dead; ++i)
        if (st->pages[g][i] >= 0) {
          if (pools[g].give_back(st->pages[g][i])) return MISUSE;
          st->pages[g][i] = -1;
        }
    }
    return OK;
  }

  int check() {
    for (size_t g = 0; g < pools.size(); ++g) {
      std::vector<int> seen(pools[g].n_pages, 0);
      long long held = 0;
      for (const Slot& st : slots)
        if (st.live)
          for (int p : st.pages[g])
            if (p >= 0) {
              if (seen[p]++) return fail(MISUSE, "group %zu: a page is held twice", g);
              ++held;
            }
      if (held + pools[g].n_free() != pools[g].n_pages)
        return fail(MISUSE, "group %zu: %lld pages are lost", g, pools[g].n_pages - pools[g].n_free() - held);
      for (int p : pools[g].free_list)
        if (seen[p]) return fail(MISUSE, "group %zu: a held page is also on the free list", g);
    }
    int n_live = 0;
    std::vector<char> is_free(n_slots, 0);
    for (int s : free_slots) is_free[s] = 1;
    for (int s = 0; s < n_slots; ++s) {
      if (slots[s].live) ++n_live;
      if (slots[s].live && is_free[s]) return fail(MISUSE, "a slot is lost or both live and free");
    }
    if (n_live + (int)free_slots.size() != n_slots) return fail(MISUSE, "a slot is lost or both live and free");
    return OK;
  }
};

inline long long align4(long long n) { return (n + 3) / 4 * 4; }

// The layout of the step buffer, in int32 elements: tokens, token_seq, token_pos [T]; seq_start [B+1]; seq_past,
// seq_slot [B]; want_rows [W]; one block table [B, width_g] per group; every array starts on a multiple of 4.
// meta: n_tokens, n_seqs, n_want, total, max_new, max_len, is_decode, n_groups, then 7 + n_groups offsets, then
// n_groups widths.
struct Layout {
  long long n_tokens, n_seqs, n_want, total;
  std::vector<long long> off;
  std::vector<long long> width;
};

Layout make_layout(long long T, long long B, long long W, const std::vector<long long>& widths) {
  Layout l{T, B, W, 0, {}, widths};
  long long at = 0;
  const long long sizes[7] = {T, T, T, B + 1, B, B, W};
  for (long long n : sizes) {
    l.off.push_back(at);
    at = align4(at + n);
  }
  for (long long w : widths) {
    l.off.push_back(at);
    at = align4(at + B * w);
  }
  l.total = std::max<long long>(at, 4);
  return l;
}

void write_meta(const Layout& l, long long max_new, long long max_len, bool is_decode, long long* meta) {
  const long long ng = (long long)l.width.size();
  meta[0] = l.n_tokens, meta[1] = l.n_seqs, meta[2] = l.n_want, meta[3] = l.total;
  meta[4] = max_new, meta[5] = max_len, meta[6] = is_decode ? 1 : 0, meta[7] = ng;
  for (size_t i = 0; i < l.off.size(); ++i) meta[8 + i] = l.off[i];
  for (long long g = 0; g < ng; ++g) meta[8 + 7 + ng + g] = l.width[g];
}

// Packs a step.  page_row(g, i, &len) gives sequence i's page list in group g.
template <typename RowFn>
int pack(long long B, const int* slots, const int* counts, const int* tokens, const int* want_counts, const int* wants,
         const long long* lengths, int n_groups, RowFn page_row, int* buf, long long cap, long long* meta) {
  long long T = 0, W = 0, max_new = 0, max_len = 0;
  bool is_decode = true;
  for (long long i = 0; i < B; ++i) {
    T += counts[i];
    W += want_counts[i] < 0 ? 1 : want_counts[i];
    max_new = std::max<long long>(max_new, counts[i]);
    max_len = std::max(max_len, lengths[i] + counts[i]);
    if (counts[i] != 1) is_decode = false;
  }
  // one width for every group: the longest sequence after this step, rounded up so that a growing sequence
  // changes the layout rarely
  const long long width = align4(std::max(1LL, pages_for(max_len)));
  Layout l = make_layout(T, B, W, std::vector<long long>((size_t)n_groups, width));
  write_meta(l, max_new, max_len, is_decode, meta);
  if (l.total > cap) return fail(TOO_SMALL, "the step buffer holds %lld elements, the step needs %lld", cap, l.total);
  std::memset(buf, 0, (size_t)l.total * sizeof(int));
  int *tok = buf + l.off[0], *tseq = buf + l.off[1], *tpos = buf + l.off[2], *start = buf + l.off[3];
  int *past = buf + l.off[4], *slot_out = buf + l.off[5], *want_rows = buf + l.off[6];
  long long at = 0, w_at = 0, wi = 0;
  for (long long i = 0; i < B; ++i) {
    start[i] = (int)at;
    past[i] = (int)lengths[i];
    slot_out[i] = slots[i];
    for (int k = 0; k < counts[i]; ++k, ++at) {
      tok[at] = tokens[at];
      tseq[at] = (int)i;
      tpos[at] = (int)(lengths[i] + k);
    }
    if (want_counts[i] < 0) {
      want_rows[w_at++] = start[i] + counts[i] - 1;
    } else {
      for (int k = 0; k < want_counts[i]; ++k) want_rows[w_at++] = start[i] + wants[wi++];
    }
  }
  start[B] = (int)at;
  for (int g = 0; g < n_groups; ++g) {
    int* tab = buf + l.off[7 + g];
    std::fill(tab, tab + B * width, -1);
    for (long long i = 0; i < B; ++i) {
      int len = 0;
      const int* row = page_row(g, i, &len);
      std::copy(row, row + std::min<long long>(len, width), tab + i * width);
    }
  }
  return OK;
}

}  // namespace

// ---------------------------------------------------------------------------
// C interface.  Functions return 0, or a code: 1 misuse of the cache, 2 a sequence would outgrow the cache's
// longest sequence, 3 no slot or page left, 4 a bad value in a step, 5 the step brings more tokens than a step
// may, 6 the step buffer is too small (meta[3] says what is needed).  llmx_host_error gives the message.
// ---------------------------------------------------------------------------
LLMX_API int llmx_host_error(char* out, int cap, long long* info) {
  std::snprintf(out, (size_t)cap, "%s", g_error.c_str());
  if (info) info[0] = g_info[0], info[1] = g_info[1];
  return (int)g_error.size();
}

LLMX_API void* llmx_alloc_new(int n_slots, int n_pages, const int* windows, int n_groups, long long max_seq_len) {
  if (n_slots <= 0 || n_pages <= 0 || n_groups <= 0) return nullptr;
  return new Allocator(n_slots, n_pages, windows, n_groups, max_seq_len);
}
LLMX_API void llmx_alloc_delete(void* a) { delete static_cast<Allocator*>(a); }
LLMX_API int llmx_alloc_acquire(void* a) { return static_cast<Allocator*>(a)->acquire(); }      // slot, or -code
LLMX_API int llmx_alloc_release(void* a, int slot) { return static_cast<Allocator*>(a)->release(slot); }
LLMX_API int llmx_alloc_reserve(void* a, int slot, long long n) { return static_cast<Allocator*>(a)->reserve(slot, n); }
LLMX_API int llmx_alloc_unreserve(void* a, int slot) { return static_cast<Allocator*>(a)->unreserve(slot); }
LLMX_API int llmx_alloc_commit(void* a, int slot, long long n) { return static_cast<Allocator*>(a)->commit(slot, n); }
LLMX_API int llmx_alloc_commit_many(void* a, int n, const int* slots, const int* counts) {
  for (int i = 0; i < n; ++i)
    if (int rc = static_cast<Allocator*>(a)->commit(slots[i], counts[i])) return rc;
  return OK;
}
LLMX_API int llmx_alloc_check(void* a) { return static_cast<Allocator*>(a)->check(); }
LLMX_API long long llmx_alloc_length(void* a, int slot) {          // -1: misuse
  Slot* st = static_cast<Allocator*>(a)->live(slot);
  return st ? st->length : -1;
}
LLMX_API long long llmx_alloc_generation(void* a, int slot) {
  Allocator* al = static_cast<Allocator*>(a);
  return (slot >= 0 && slot < al->n_slots) ? al->slots[slot].generation : -1;
}
LLMX_API int llmx_alloc_n_free_slots(void* a) { return (int)static_cast<Allocator*>(a)->free_slots.size(); }
LLMX_API int llmx_alloc_n_free_pages(void* a, int group) { return static_cast<Allocator*>(a)->pools[group].n_free(); }
// Copies the slot's page list of a group into out (up to cap entries); returns its length, or -1 on misuse.
LLMX_API int llmx_alloc_page_row(void* a, int slot, int group, int* out, int cap) {
  Allocator* al = static_cast<Allocator*>(a);
  Slot* st = al->live(slot);
  if (!st || group < 0 || group >= (int)al->pools.size()) return -1;
  const auto& row = st->pages[group];
  std::copy(row.begin(), row.begin() + std::min<size_t>(row.size(), (size_t)cap), out);
  return (int)row.size();
}

// Packs a step whose lengths and page lists the caller already has (rows: for each group, for each sequence, its
// page list; row_len the lengths, row_off the start of each list in `rows`).
LLMX_API int llmx_pack_step(int n_seqs, const int* slots, const int* counts, const int* tokens, const int* want_counts,
                            const int* wants, const long long* lengths, int n_groups, const int* rows,
                            const long long* row_off, const int* row_len, int* buf, long long cap, long long* meta) {
  auto page_row = [&](int g, long long i, int* len) {
    *len = row_len[(long long)g * n_seqs + i];
    return rows + row_off[(long long)g * n_seqs + i];
  };
  return pack(n_seqs, slots, counts, tokens, want_counts, wants, lengths, n_groups, page_row, buf, cap, meta);
}

// One step, from the entries to the packed buffer: every check that can refuse the step, then the reservation of
// pages for every sequence (taken back if one of them does not fit), then the packing.  want_counts[i] < 0: the
// last token of sequence i.  A refused step leaves the cache as it was.
LLMX_API int llmx_plan_step(void* a, int n_seqs, const int* slots, const int* counts, const int* tokens,
                            const int* want_counts, const int* wants, int vocab, long long max_step_tokens,
                            int n_groups, int* buf, long long cap, long long* meta) {
  Allocator* al = static_cast<Allocator*>(a);
  if (n_seqs <= 0) return fail(BAD_VALUE, "a step needs at least one sequence");
  std::vector<char> seen((size_t)al->n_slots, 0);
  std::vector<long long> lengths((size_t)n_seqs);
  long long total = 0, ti = 0, wi = 0;
  for (int i = 0; i < n_seqs; ++i) {
    const int slot = slots[i];
    if (slot >= 0 && slot < al->n_slots && seen[slot]) return fail(MISUSE, "slot %d appears twice in one step", slot);
    Slot* st = al->live(slot);
    if (!st) return MISUSE;
    seen[slot] = 1;
    if (counts[i] <= 0) return fail(BAD_VALUE, "slot %d brings no token", slot);
    for (int k = 0; k < counts[i]; ++k, ++ti)
      if (tokens[ti] < 0 || tokens[ti] >= vocab)
        return fail(BAD_VALUE, "token id %d is outside the vocabulary of %d", tokens[ti], vocab);
    for (int k = 0; k < want_counts[i]; ++k, ++wi)
      if (wants[wi] < 0 || wants[wi] >= counts[i])
        return fail(BAD_VALUE, "slot %d: wanted place %d is outside its %d tokens", slot, wants[wi], counts[i]);
    total += counts[i];
    lengths[i] = st->length;
  }
  if (total > max_step_tokens) {
    g_info[0] = total, g_info[1] = max_step_tokens;
    return fail(OVERFLOW_STEP, "%lld tokens do not fit the step limit (max_step_tokens) of %lld", total, max_step_tokens);
  }
  int done = 0, rc = OK;
  for (; done < n_seqs; ++done)
    if ((rc = al->reserve(slots[done], counts[done])) != OK) break;
  if (rc == OK) {
    auto page_row = [&](int g, long long i, int* len) {
      const auto& row = al->slots[slots[i]].pages[g];
      *len = (int)row.size();
      return row.data();
    };
    rc = pack(n_seqs, slots, counts, tokens, want_counts, wants, lengths.data(), n_groups, page_row, buf, cap, meta);
  }
  if (rc != OK) {
    const std::string keep = g_error;
    for (int i = 0; i < done; ++i) al->unreserve(slots[i]);
    g_error = keep;
  }
  return rc;
}
