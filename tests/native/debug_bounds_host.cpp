// Host-side check of the destination rule that debug builds of the Tier-1 device code apply
// (aboleth/debug_bounds.h is plain C++ for exactly this purpose).
#include <cstdio>

#include "aboleth/debug_bounds.h"

int main() {
    using aboleth::debug::Bounds;
    using aboleth::debug::Window;
    using aboleth::debug::inside;
    const Window windows[2] = {{0x1000, 0x100}, {0xffffffffffffff00ull, 0x80}};
    const Bounds bounds{windows, 2, nullptr};
    int failures = 0;
    const auto expect = [&](bool got, bool want, const char *what) {
        if (got != want) {
            std::fprintf(stderr, "debug_bounds: %s\n", what);
            ++failures;
        }
    };
    expect(inside(bounds, 0x1000, 0x100), true, "the whole window is writable");
    expect(inside(bounds, 0x10f8, 8), true, "the last word of a window is writable");
    expect(inside(bounds, 0x10f9, 8), false, "a write that straddles the end is refused");
    expect(inside(bounds, 0xfff, 2), false, "a write that starts before the base is refused");
    expect(inside(bounds, 0x2000, 1), false, "an address in no window is refused");
    expect(inside(bounds, 0x2000, 0), true, "an empty write is always fine");
    expect(inside(bounds, 0xffffffffffffff00ull, 0x80), true, "a window near the top of the address space works");
    expect(inside(bounds, 0xfffffffffffffff8ull, 16), false, "a range that wraps around is refused");
    expect(inside(Bounds{}, 0xdead, 64), true, "no windows means nothing is checked");
    expect(inside(Bounds{windows, 0, nullptr}, 0xdead, 64), true, "a count of zero means nothing is checked");
    std::printf("failures: %d\n", failures);
    return failures == 0 ? 0 : 1;
}
