// Native page bookkeeping (host only): the id pool, reference counts for shared pages, and the
// per-instance ownership / out-of-memory policy / export-import of the reference's resource manager,
// restated for KV pages of ONE device group (the reference keeps one such pool per data-parallel
// group, runtime/src/model/resource.rs:83-87).
//
//   * ids: always the smallest free id; ids that were never handed out cannot be released; once more
//     than 1000 ids are free, a free block at the tail is folded back into the never-allocated range
//     (runtime/src/utils.rs:42-158);
//   * instances own sets of pages; an allocation that does not fit terminates instances that started
//     AFTER the requester, newest first, until it fits, and fails if that is not enough
//     (resource.rs:112-319);
//   * export moves pages from an instance to a name, import reads them, release_exported frees them
//     (resource.rs:356-451);
//   * reference counts are this library's addition for forked contexts that share full pages
//     (the reference's SDK counts them per context, sdk/rust/inferlet/src/forward.rs:28-55): a page
//     goes back to the id pool when its last reference is dropped.
//
// Not thread safe: the reference drives its manager from one task, and so must the caller here.
#include <stdint.h>
#include <string.h>

#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "common.cuh"

namespace {

struct IdPool {
  uint32_t next = 0;
  uint32_t cap = 0;
  std::set<uint32_t> free_ids;

  size_t available() const { return free_ids.size() + (size_t)(cap - next); }
  bool acquire(uint32_t *id) {
    if (!free_ids.empty()) {
      *id = *free_ids.begin();
      free_ids.erase(free_ids.begin());
      return true;
    }
    if (next < cap) {
      *id = next++;
      return true;
    }
    return false;
  }
  bool release(uint32_t id) {
    if (id >= next) return false;
    free_ids.insert(id);
    return true;
  }
  void compact_if_large() {
    if (free_ids.size() <= 1000) return;
    while (!free_ids.empty() && *free_ids.rbegin() == next - 1) {
      free_ids.erase(std::prev(free_ids.end()));
      --next;
    }
  }
};

struct Instance {
  std::unordered_set<uint32_t> pages;
  uint64_t started = 0;  // logical clock of the first allocation (the reference uses Instant::now)
  bool has_started = false;
};

}  // namespace

struct piekv_page_manager {
  IdPool ids;
  std::vector<int32_t> refs;
  std::unordered_map<uint64_t, Instance> inst;
  std::map<std::string, std::vector<uint32_t>> exported;
  uint64_t clock = 0;
  std::vector<uint64_t> last_victims;
};

using piekv::set_error;

extern "C" piekv_page_manager *piekv_pages_create(int32_t num_pages) {
  if (num_pages < 0) {
    set_error("pages_create: negative capacity");
    return nullptr;
  }
  piekv_page_manager *m = new piekv_page_manager();
  m->ids.cap = (uint32_t)num_pages;
  m->refs.assign((size_t)num_pages, 0);
  return m;
}

extern "C" void piekv_pages_destroy(piekv_page_manager *m) { delete m; }

extern "C" int32_t piekv_pages_available(const piekv_page_manager *m) { return m ? (int32_t)m->ids.available() : 0; }

extern "C" int32_t piekv_pages_refcount(const piekv_page_manager *m, int32_t page) {
  if (!m || page < 0 || (size_t)page >= m->refs.size()) return -1;
  return m->refs[(size_t)page];
}

extern "C" int32_t piekv_pages_owned(const piekv_page_manager *m, uint64_t instance) {
  if (!m) return 0;
  auto it = m->inst.find(instance);
  return it == m->inst.end() ? 0 : (int32_t)it->second.pages.size();
}

// Drop one reference of a page the caller no longer lists anywhere; back to the id pool at zero.
static bool unref(piekv_page_manager *m, uint32_t page) {
  if ((size_t)page >= m->refs.size() || m->refs[page] <= 0) return false;
  if (--m->refs[page] == 0) m->ids.release(page);
  return true;
}

static void cleanup_instance(piekv_page_manager *m, uint64_t instance) {
  auto it = m->inst.find(instance);
  if (it == m->inst.end()) return;
  for (uint32_t p : it->second.pages) unref(m, p);
  m->inst.erase(it);
  m->ids.compact_if_large();
}

extern "C" int piekv_pages_alloc(piekv_page_manager *m, uint64_t instance, int32_t count, int32_t *out) {
  PIEKV_REQUIRE(m != nullptr && count >= 0 && (count == 0 || out != nullptr), "pages_alloc: bad arguments");
  m->last_victims.clear();
  Instance &me = m->inst[instance];
  if (m->ids.available() < (size_t)count) {
    // out-of-memory policy: newest instances that started after the requester go first
    if (!me.has_started) {
      set_error("pages_alloc: out of pages and the requesting instance has no start time");
      return PIEKV_STATUS_OUT_OF_PAGES;
    }
    while (m->ids.available() < (size_t)count) {
      uint64_t victim = 0, best = 0;
      bool found = false;
      for (auto &kv : m->inst) {
        if (kv.first == instance || !kv.second.has_started || kv.second.started <= me.started) continue;
        if (!found || kv.second.started > best) {
          found = true;
          best = kv.second.started;
          victim = kv.first;
        }
      }
      if (!found) {
        set_error("pages_alloc: not enough pages after terminating all newer instances");
        return PIEKV_STATUS_OUT_OF_PAGES;
      }
      cleanup_instance(m, victim);
      m->last_victims.push_back(victim);
    }
  }
  Instance &self = m->inst[instance];  // (the map may have rehashed while victims were erased)
  if (!self.has_started) {
    self.has_started = true;
    self.started = ++m->clock;
  }
  for (int32_t i = 0; i < count; ++i) {
    uint32_t id = 0;
    m->ids.acquire(&id);  // cannot fail: available() >= count was established above
    m->refs[id] = 1;
    self.pages.insert(id);
    out[i] = (int32_t)id;
  }
  return 0;
}

extern "C" int32_t piekv_pages_last_victims(const piekv_page_manager *m, uint64_t *out, int32_t max_count) {
  if (!m) return 0;
  const int32_t n = (int32_t)m->last_victims.size();
  for (int32_t i = 0; i < n && i < max_count; ++i) out[i] = m->last_victims[(size_t)i];
  return n;
}

extern "C" int piekv_pages_free(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count) {
  PIEKV_REQUIRE(m != nullptr && count >= 0 && (count == 0 || pages != nullptr), "pages_free: bad arguments");
  auto it = m->inst.find(instance);
  PIEKV_REQUIRE(it != m->inst.end(), "pages_free: instance %llu holds no pages", (unsigned long long)instance);
  for (int32_t i = 0; i < count; ++i) {
    // pages the instance does not hold are skipped, as in the reference (resource.rs:248-252)
    if (pages[i] >= 0 && it->second.pages.erase((uint32_t)pages[i])) unref(m, (uint32_t)pages[i]);
  }
  m->ids.compact_if_large();
  return 0;
}

// `instance` becomes a co-owner of pages some other instance (or an export) already holds.
extern "C" int piekv_pages_share(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count) {
  PIEKV_REQUIRE(m != nullptr && count >= 0 && (count == 0 || pages != nullptr), "pages_share: bad arguments");
  for (int32_t i = 0; i < count; ++i)
    PIEKV_REQUIRE(pages[i] >= 0 && (size_t)pages[i] < m->refs.size() && m->refs[(size_t)pages[i]] > 0,
                  "pages_share: page %d is not allocated", pages[i]);
  Instance &self = m->inst[instance];
  if (!self.has_started) {
    self.has_started = true;
    self.started = ++m->clock;
  }
  for (int32_t i = 0; i < count; ++i) {
    if (self.pages.insert((uint32_t)pages[i]).second) ++m->refs[(size_t)pages[i]];
  }
  return 0;
}

extern "C" int piekv_pages_cleanup(piekv_page_manager *m, uint64_t instance) {
  PIEKV_REQUIRE(m != nullptr, "pages_cleanup: null manager");
  cleanup_instance(m, instance);
  return 0;
}

extern "C" int piekv_pages_export(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count,
                                  const char *name) {
  PIEKV_REQUIRE(m != nullptr && name != nullptr && count >= 0 && (count == 0 || pages != nullptr),
                "pages_export: bad arguments");
  auto it = m->inst.find(instance);
  PIEKV_REQUIRE(it != m->inst.end(), "pages_export: instance %llu holds no pages", (unsigned long long)instance);
  for (int32_t i = 0; i < count; ++i)
    PIEKV_REQUIRE(pages[i] >= 0 && it->second.pages.count((uint32_t)pages[i]),
                  "pages_export: page %d is not allocated to instance %llu", pages[i], (unsigned long long)instance);
  PIEKV_REQUIRE(!m->exported.count(name), "pages_export: export name '%s' exists", name);
  {
    // A page listed twice would be released twice later and take a co-holder's reference with it.
    std::unordered_set<uint32_t> seen;
    for (int32_t i = 0; i < count; ++i)
      PIEKV_REQUIRE(seen.insert((uint32_t)pages[i]).second, "pages_export: page %d is listed twice", pages[i]);
  }
  std::vector<uint32_t> v;
  for (int32_t i = 0; i < count; ++i) {
    it->second.pages.erase((uint32_t)pages[i]);  // ownership (and the reference) moves to the name
    v.push_back((uint32_t)pages[i]);
  }
  m->exported.emplace(name, std::move(v));
  return 0;
}

extern "C" int32_t piekv_pages_import(const piekv_page_manager *m, const char *name, int32_t *out, int32_t max_count) {
  if (!m || !name) return -1;
  auto it = m->exported.find(name);
  if (it == m->exported.end()) {
    set_error("pages_import: export '%s' not found", name);
    return -1;
  }
  const int32_t n = (int32_t)it->second.size();
  for (int32_t i = 0; i < n && i < max_count; ++i) out[i] = (int32_t)it->second[(size_t)i];
  return n;
}

extern "C" int piekv_pages_release_exported(piekv_page_manager *m, const char *name) {
  PIEKV_REQUIRE(m != nullptr && name != nullptr, "pages_release_exported: bad arguments");
  auto it = m->exported.find(name);
  PIEKV_REQUIRE(it != m->exported.end(), "pages_release_exported: export '%s' not found", name);
  for (uint32_t p : it->second) unref(m, p);
  m->exported.erase(it);
  m->ids.compact_if_large();
  return 0;
}
