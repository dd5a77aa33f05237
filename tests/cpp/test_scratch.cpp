// Host-only check of the grow-on-demand bookkeeping (prism_engine_b200/csrc/scratch.hpp) with an
// allocator that can be told to fail: after a failed allocation the buffer must read as empty, so a
// later, smaller request allocates again instead of handing a null pointer to a kernel.
#include <cstdio>
#include <cstdlib>

#include "../../prism_engine_b200/csrc/scratch.hpp"

struct FakeAlloc {
    int fail_next_acquire = 0, fail_sync = 0;
    int acquires = 0, releases = 0, syncs = 0, live = 0;
    int sync() { syncs++; return fail_sync ? 7 : 0; }
    int release(void *p) { releases++; live--; free(p); return 0; }
    int acquire(void **p, size_t bytes) {
        acquires++;
        if (fail_next_acquire) { fail_next_acquire--; return 2; }
        *p = malloc(bytes);
        live++;
        return *p ? 0 : 2;
    }
};

#define CHECK(c) do { if (!(c)) { printf("FAIL line %d: %s\n", __LINE__, #c); return 1; } } while (0)

int main() {
    using namespace prism;
    FakeAlloc al;
    GrowBuf b;
    bool grew = false;
    CHECK(grow_buf(al, b, 100, 4, &grew) == 0 && grew && b.ptr && b.count >= 100 && al.live == 1);
    CHECK(b.count * 4 % 256 == 0);                                   // rounded to 256 bytes
    void *first = b.ptr;
    CHECK(grow_buf(al, b, 50, 4, &grew) == 0 && !grew && b.ptr == first && al.acquires == 1);   // fits: untouched
    // growth that fails: the old buffer is gone, the record says so
    al.fail_next_acquire = 1;
    CHECK(grow_buf(al, b, 1000, 4, &grew) == 2 && !grew);
    CHECK(b.ptr == nullptr && b.count == 0 && al.live == 0);
    // the smaller request that used to slip through `want <= have` now allocates
    CHECK(grow_buf(al, b, 50, 4, &grew) == 0 && grew && b.ptr && b.count >= 50 && al.live == 1);
    // a failing synchronise leaves the buffer as it was (nothing freed yet)
    al.fail_sync = 1;
    void *kept = b.ptr;
    const size_t kept_n = b.count;
    CHECK(grow_buf(al, b, 5000, 4, &grew) == 7 && b.ptr == kept && b.count == kept_n && al.live == 1);
    al.fail_sync = 0;
    CHECK(grow_buf(al, b, 5000, 2, &grew) == 0 && b.count >= 5000 && al.live == 1 && al.releases == 2);
    al.release(b.ptr);
    printf("ok\n");
    return 0;
}
