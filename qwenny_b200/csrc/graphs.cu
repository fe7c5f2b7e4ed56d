// Host-only check of the step-graph cache policy (graphs.h) with fakes behind its hooks: no CUDA call.
#include "graphs.h"
#include <set>
#include "measure.h"

extern "C" int qb_graph_cache_selftest(void) {
    using Cache = qb::GraphCache<int, int>;
    size_t free_now = (size_t)1 << 30, released = 0;
    int syncs = 0;
    std::set<int> destroyed;
    Cache::Hooks hk;
    hk.free_mem = [&]() { return free_now; };
    hk.destroy = [&](int& g) { destroyed.insert(g); };
    hk.sync = [&]() { syncs++; };
    hk.release = [&](size_t bytes) { released += bytes; return bytes; };
    const size_t FLOOR = (size_t)128 << 20;
    Cache c(hk, FLOOR);
    // plenty of memory: no cap, every graph kept
    for (int k = 0; k < 40; k++) {
        if (c.find(k)) return 1;
        c.make_room();
        c.insert(k, 100 + k);
    }
    if (c.size() != 40 || c.cap() != Cache::NO_CAP || !destroyed.empty()) return 2;
    // memory short at the next capture: the cap becomes what is held, the least recently used graph goes
    for (int k = 1; k < 40; k++)
        if (!c.find(k)) return 3;  // key 0 is now the oldest
    free_now = (size_t)100 << 20;
    if (c.find(40)) return 4;
    c.make_room();
    c.insert(40, 140);
    if (c.cap() != 40 || c.size() != 40 || !destroyed.count(100) || c.holds(0) || syncs == 0) return 5;
    if (released != 0) return 6;  // above half the floor: the pool keeps its pages
    // the same free memory again does not lower the cap; less does, by a sixteenth
    c.find(41); c.make_room(); c.insert(41, 141);
    if (c.cap() != 40 || c.size() != 40) return 7;
    free_now = (size_t)90 << 20;
    c.find(42); c.make_room(); c.insert(42, 142);
    if (c.cap() != 40 - 40 / 16 || c.size() != c.cap()) return 8;
    // below half the floor the pool gives pages back
    free_now = (size_t)40 << 20;
    c.find(43); c.make_room(); c.insert(43, 143);
    if (released != FLOOR - free_now) return 9;
    // a capture without memory: three quarters kept, and the cache goes on working
    const size_t held = c.size();
    c.find(44); c.make_room();
    c.on_out_of_memory();
    if (c.cap() != (held - 1) * 3 / 4 && c.cap() != held * 3 / 4) return 10;
    if (c.size() >= c.cap() + 1) return 11;
    // a used graph survives eviction ahead of unused ones
    if (!c.find(43)) return 12;
    for (int k = 50; k < 50 + 64; k++) { c.find(k); c.make_room(); c.insert(k, 100 + k); c.find(43); }
    if (!c.holds(43)) return 13;
    // retain drops what the predicate refuses, clear the rest
    const size_t before = c.size();
    c.retain([](const int& k) { return k != 43; });
    if (c.size() != before - 1 || c.holds(43)) return 14;
    c.clear();
    if (c.size() != 0) return 15;
    return 0;
}
