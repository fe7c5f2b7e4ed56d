"""The cache of captured step graphs (csrc/graphs.h) on a CPU: its hooks take fakes, a small C++ driver
(tests/graph_cache_policy.cpp, compiled here with g++) replays a script of steps, and the state after every step must be
that of the policy of the reference's host (Graphs::run, make_room, evict: src/cuda/core.rs:1151-1250), restated below."""
import os
import random
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FLOOR = 128 << 20
NO_CAP = float("inf")


class Policy:
    """What the reference's host keeps, step by step. `graphs`: key -> tick of its last run."""

    def __init__(self):
        self.graphs, self.tick, self.cap, self.low = {}, 0, NO_CAP, NO_CAP
        self.destroyed = self.syncs = self.asked = 0

    def evict(self):  # core.rs:1235-1250: the least recently used go until fewer than the cap are kept
        if len(self.graphs) < self.cap:
            return
        self.syncs += 1
        n = len(self.graphs) + 1 - max(self.cap, 1)
        for k in sorted(self.graphs, key=lambda k: self.graphs[k])[:n]:
            del self.graphs[k]
            self.destroyed += 1

    def make_room(self, free):  # core.rs:1198-1233
        if free < min(FLOOR, self.low) and self.graphs:
            n = min(self.cap, len(self.graphs))
            self.cap = n if self.cap == NO_CAP else n - n // 16
            self.low = free
        if len(self.graphs) >= self.cap:
            self.cap = max(self.cap, 1)
            self.evict()
        if free < FLOOR // 2:
            self.asked += FLOOR - free

    def run(self, key, free, oom):  # core.rs:1151-1192
        self.tick += 1
        if key in self.graphs:
            self.graphs[key] = self.tick
            return "hit"
        self.make_room(free)
        if oom:
            self.cap = len(self.graphs) * 3 // 4
            self.evict()
            return "oom"
        self.graphs[key] = self.tick
        return "new"

    def retain(self, keep):  # core.rs:1146-1148 (the library also waits for the device once before it drops any)
        gone = [k for k in self.graphs if not keep(k)]
        if gone:
            self.syncs += 1
        for k in gone:
            del self.graphs[k]
            self.destroyed += 1

    def state(self, what):
        cap = -1 if self.cap == NO_CAP else self.cap
        return " ".join([what, str(cap), str(self.destroyed), str(self.syncs), str(self.asked)] +
                        [str(k) for k in sorted(self.graphs)])


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("graph_cache") / "policy")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "qwenny_b200", "csrc"),
                    os.path.join(ROOT, "tests", "graph_cache_policy.cpp"), "-o", exe], check=True)
    return exe


def replay(driver, ops):
    text = "".join(" ".join(str(x) for x in op) + "\n" for op in ops)
    got = subprocess.run([driver], input=text, capture_output=True, text=True, check=True).stdout.splitlines()
    p, want = Policy(), []
    for op in ops:
        if op[0] == "run":
            want.append(p.state(p.run(op[1], op[2], op[3])))
        elif op[0] == "retain_even":
            p.retain(lambda k: k % 2 == 0)
            want.append(p.state("ok"))
        else:
            p.retain(lambda k: False)
            want.append(p.state("ok"))
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g == w, f"after op {i} {ops[i]}: library '{g}', policy '{w}'"
    return got


def test_unbounded_while_memory_is_plentiful(driver):
    ops = [("run", k % 50, 4 << 30, 0) for k in range(200)]
    last = replay(driver, ops)[-1].split()
    assert last[1] == "-1" and len(last) - 5 == 50 and last[2] == "0"


def test_cap_set_below_the_floor_then_lowered_as_memory_falls_and_lru_goes(driver):
    ops = [("run", k, 1 << 30, 0) for k in range(32)]
    ops += [("run", 0, 0, 0), ("run", 1, 0, 0)]                        # replays: keys 0 and 1 are now the youngest
    ops += [("run", 100, 100 << 20, 0)]                                # below the floor: the cap becomes what is held (32)
    ops += [("run", 101, 100 << 20, 0)]                                # not lower than before: the cap stays
    ops += [("run", 102, 90 << 20, 0)]                                 # lower: the cap loses a sixteenth
    ops += [("run", 103, 60 << 20, 0)]                                 # below half the floor: pages asked back as well
    got = replay(driver, ops)
    assert got[34].split()[1] == "32" and got[35].split()[1] == "32" and got[36].split()[1] == "30"
    held = set(got[36].split()[5:])
    assert {"0", "1", "100", "101", "102"} <= held and "2" not in held and "3" not in held
    assert int(got[37].split()[4]) == (128 << 20) - (60 << 20)


def test_a_capture_without_memory_keeps_three_quarters(driver):
    ops = [("run", k, 1 << 30, 0) for k in range(16)] + [("run", 99, 1 << 30, 1)]
    got = replay(driver, ops)
    f = got[-1].split()
    assert f[0] == "oom" and f[1] == "12" and len(f) - 5 == 11 and "99" not in f[5:]
    # with nothing held the cap is 0: the next capture still gets one graph's room
    got = replay(driver, [("run", 5, 1 << 30, 1), ("run", 6, 1 << 30, 0), ("run", 7, 1 << 30, 0)])
    assert got[0].split()[1] == "0" and got[2].split()[5:] == ["7"]


def test_retain_and_clear(driver):
    ops = [("run", k, 1 << 30, 0) for k in range(10)] + [("retain_even",), ("run", 3, 1 << 30, 0), ("clear",), ("clear",)]
    got = replay(driver, ops)
    assert got[10].split()[5:] == ["0", "2", "4", "6", "8"] and got[12].split()[5:] == []
    assert got[12].split()[3] == got[13].split()[3]                    # nothing to drop: no wait for the device


@pytest.mark.parametrize("seed", range(6))
def test_random_scripts_follow_the_policy(driver, seed):
    rng = random.Random(seed)
    free, ops = 1 << 30, []
    for _ in range(1500):
        r = rng.random()
        if r < 0.01:
            ops.append(("retain_even",))
        elif r < 0.013:
            ops.append(("clear",))
        else:
            if rng.random() < 0.3:
                free = max(1 << 20, free - rng.randrange(0, 24 << 20))
            if rng.random() < 0.02:
                free += rng.randrange(0, 64 << 20)
            ops.append(("run", rng.randrange(0, 60) if rng.random() < 0.8 else rng.randrange(0, 400), free,
                        int(free < (96 << 20) and rng.random() < 0.05)))
    replay(driver, ops)
