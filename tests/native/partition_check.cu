// Host-side check of the step partition that the streaming tensor-core kernels use (TsSegs, csrc/tc_stream.cuh):
// every (tile, step) is owned by exactly one CTA, a CTA's shared segments come first and are at most two, cta_of() names
// the owner of every left-over step, and a CTA's two exchange slots are distinct.  Runs on the CPU; no GPU code is launched.
#include <cstdio>
#include <vector>

#include "tc_stream.cuh"

using sbvr::TsSegs;

static int check(int NT, int KBS, int G) {
    std::vector<int> owner((size_t)NT * KBS, -1);
    long long total = 0;
    for (int c = 0; c < G; ++c) {
        TsSegs sg;
        sg.init(NT, KBS, (unsigned)G, (unsigned)c);
        int nshared = 0, steps = 0;
        bool whole_seen = false;
        int slots_used[2] = {-1, -1};
        for (int q = 0; q < sg.nseg; ++q) {
            const int tile = sg.tile(q), k0 = sg.k0(q), k1 = sg.k1(q);
            if (tile < 0 || tile >= NT || k0 < 0 || k1 > KBS || k0 >= k1) return 1;
            if (sg.shared(q)) {
                if (whole_seen) return 2;                       // shared segments come first
                if (++nshared > 2) return 3;
                const int rt = tile - sg.rem_tile0;
                if (rt < 0) return 4;
                for (int k = k0; k < k1; ++k)
                    if (sg.cta_of((unsigned)(rt * KBS + k)) != c) return 5;
                const int sl = sg.slot_of((unsigned)c, rt);
                if (sl != 0 && sl != 1) return 6;
                if (slots_used[sl] >= 0) return 7;              // two shared segments of a CTA use different slots
                slots_used[sl] = rt;
            } else {
                whole_seen = true;
                if (k0 != 0 || k1 != KBS) return 8;
            }
            for (int k = k0; k < k1; ++k) {
                int& o = owner[(size_t)tile * KBS + k];
                if (o != -1) return 9;                          // a step owned twice
                o = c;
                ++steps;
            }
        }
        if (steps != sg.steps) return 10;
        total += steps;
    }
    if (total != (long long)NT * KBS) return 11;
    for (int o : owner)
        if (o < 0) return 12;                                   // a step nobody owns
    // the first owner of every left-over tile exists and the owners appear in ascending order
    TsSegs sg;
    sg.init(NT, KBS, (unsigned)G, 0u);
    const int R = NT - sg.rem_tile0;
    for (int rt = 0; rt < R; ++rt) {
        int prev = -1;
        for (int k = 0; k < KBS; ++k) {
            const int cc = sg.cta_of((unsigned)(rt * KBS + k));
            if (cc < 0 || cc >= G || cc < prev) return 13;
            if (owner[(size_t)(sg.rem_tile0 + rt) * KBS + k] != cc) return 14;
            prev = cc;
        }
    }
    return 0;
}

int main() {
    int bad = 0, cases = 0;
    const int grids[] = {1, 2, 3, 7, 32, 43, 112, 128, 132, 148};
    for (int G : grids)
        for (int KBS = 1; KBS <= 56; KBS += (KBS < 8 ? 1 : 7))
            for (int NT = 1; NT <= 4 * G + 5; NT += (NT < 20 ? 1 : 13)) {
                if ((long long)NT * KBS >= (1 << 24)) continue;
                ++cases;
                const int rc = check(NT, KBS, G);
                if (rc) {
                    std::printf("FAIL code %d: NT=%d KBS=%d G=%d\n", rc, NT, KBS, G);
                    if (++bad > 10) return 1;
                }
            }
    // the shapes of the benchmark: (tiles or tile groups, steps, CTAs)
    const int shapes[][3] = {{448, 8, 148}, {448, 16, 148}, {128, 8, 128}, {128, 28, 128}, {32, 8, 32}, {150, 16, 148},
                             {43, 16, 148}, {43, 56, 148}, {11, 16, 148}, {896, 16, 148}, {4008, 16, 148}};
    for (auto& s : shapes) {
        ++cases;
        const int rc = check(s[0], s[1], s[2]);
        if (rc) {
            std::printf("FAIL code %d: NT=%d KBS=%d G=%d\n", rc, s[0], s[1], s[2]);
            ++bad;
        }
    }
    std::printf("%d cases, %d failures\n", cases, bad);
    return bad ? 1 : 0;
}
