// Bookkeeping of the context's grow-on-demand device buffers, kept free of CUDA so the failure
// paths can be exercised on a host with a fake allocator (tests/cpp/test_scratch.cpp).
#pragma once

#include <cstddef>

namespace prism {

// A device buffer that only ever grows.  `count` is in elements of `elem_size` bytes and is the
// single source of truth: it is zero whenever `ptr` is null.
struct GrowBuf {
    void *ptr = nullptr;
    size_t count = 0;
};

// Makes `b` hold at least `want` elements.  The allocator provides
//   int sync()                    wait for work that may still use the old buffer (0 = ok)
//   int release(void *p)          free a buffer (0 = ok)
//   int acquire(void **p, size_t bytes)   allocate (0 = ok, *p untouched or null on failure)
// Returns 0, or the allocator's error code with `b` left EMPTY (null, 0 elements): after a failed
// allocation the old buffer is already gone, so a later, smaller request must allocate again
// instead of being waved through against a stale size.
template <typename Alloc>
int grow_buf(Alloc &al, GrowBuf &b, size_t want, size_t elem_size, bool *grew = nullptr) {
    if (grew) *grew = false;
    if (want <= b.count) return 0;
    int rc = al.sync();
    if (rc) return rc;
    void *old = b.ptr;
    b.ptr = nullptr;
    b.count = 0;
    if (old && (rc = al.release(old)) != 0) return rc;
    const size_t bytes = (want * elem_size + 255) / 256 * 256;
    void *p = nullptr;
    rc = al.acquire(&p, bytes);
    if (rc || !p) return rc ? rc : -1;
    b.ptr = p;
    b.count = bytes / elem_size;
    if (grew) *grew = true;
    return 0;
}

}  // namespace prism
