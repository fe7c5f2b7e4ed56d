// Drives qb::GraphCache (csrc/graphs.h) with fakes behind its hooks, for tests/test_graph_cache_cpu.py: reads one
// operation per line from stdin and prints the cache's state after each.
//   run <key> <free bytes> <oom 0|1>   a step of that key: replayed if held, else make_room, then a capture that
//                                      succeeds (insert) or finds no memory (on_out_of_memory), as the model's runner does
//   retain_even                        drop the graphs with odd keys
//   clear
// Output per line: hit|new|oom|ok, the cap (-1: none), graphs destroyed so far, syncs so far, bytes asked back from
// the pool so far, then the held keys in ascending order.
#include <cstdio>
#include <cstring>
#include <set>
#include <string>

#include "graphs.h"

int main() {
    size_t free_now = 0, destroyed = 0, syncs = 0, asked = 0;
    std::set<int> alive;
    using Cache = qb::GraphCache<int, int>;
    Cache::Hooks hk;
    hk.free_mem = [&]() { return free_now; };
    hk.destroy = [&](int& g) { destroyed++; alive.erase(g); };
    hk.sync = [&]() { syncs++; };
    hk.release = [&](size_t bytes) { asked += bytes; return bytes; };
    Cache cache(hk, (size_t)128 << 20);
    char line[256];
    while (fgets(line, sizeof line, stdin)) {
        int key = 0, oom = 0;
        unsigned long long fr = 0;
        const char* what = "ok";
        if (sscanf(line, "run %d %llu %d", &key, &fr, &oom) == 3) {
            if (cache.find(key)) what = "hit";
            else {
                free_now = (size_t)fr;
                cache.make_room();
                if (oom) { cache.on_out_of_memory(); what = "oom"; }
                else { cache.insert(key, key); alive.insert(key); what = "new"; }
            }
        } else if (!strncmp(line, "retain_even", 11)) cache.retain([](const int& k) { return k % 2 == 0; });
        else if (!strncmp(line, "clear", 5)) cache.clear();
        else continue;
        printf("%s %lld %zu %zu %zu", what, cache.cap() == Cache::NO_CAP ? -1LL : (long long)cache.cap(), destroyed, syncs, asked);
        for (int k : alive) {
            if (!cache.holds(k)) { printf(" LOST%d", k); }
            printf(" %d", k);
        }
        if (alive.size() != cache.size()) printf(" SIZE%zu", cache.size());
        printf("\n");
    }
    return 0;
}
