// cxx_linkage.cpp — the runtime helpers under the C++-linkage names of the reference.
//
// xpu/src/tq_common.hpp:212-216 declares tq_dev_alloc, tq_dev_free, tq_h2d, tq_d2h and
// tq_dev_zero outside its extern "C" block, so objects compiled against that header (the
// reference's probes, e.g. xpu/probe/fanout_bench.cpp:20, and its layer bodies) ask the
// linker for the Itanium-mangled names. This library's own header exports the five helpers
// with C linkage for FFI bindings; a C++ function of the same name and signature cannot be
// declared beside an extern "C" one, so the mangled symbols are given here as assembler
// labels of differently named forwarders. This file must not include tq_w4a8.h.
#include <stddef.h>

extern "C" {
void *tq_dev_alloc(size_t bytes, const char *what);
void tq_dev_free(void *p);
void tq_h2d(void *dst, const void *src, size_t bytes);
void tq_d2h(void *dst, const void *src, size_t bytes);
void tq_dev_zero(void *dst, size_t bytes);
}

#define TQ_EXPORT __attribute__((visibility("default")))

TQ_EXPORT void *tq_cxx_dev_alloc(size_t bytes, const char *what) asm("_Z12tq_dev_allocmPKc");
TQ_EXPORT void tq_cxx_dev_free(void *p) asm("_Z11tq_dev_freePv");
TQ_EXPORT void tq_cxx_h2d(void *dst, const void *src, size_t bytes) asm("_Z6tq_h2dPvPKvm");
TQ_EXPORT void tq_cxx_d2h(void *dst, const void *src, size_t bytes) asm("_Z6tq_d2hPvPKvm");
TQ_EXPORT void tq_cxx_dev_zero(void *dst, size_t bytes) asm("_Z11tq_dev_zeroPvm");

void *tq_cxx_dev_alloc(size_t bytes, const char *what) { return tq_dev_alloc(bytes, what); }
void tq_cxx_dev_free(void *p) { tq_dev_free(p); }
void tq_cxx_h2d(void *dst, const void *src, size_t bytes) { tq_h2d(dst, src, bytes); }
void tq_cxx_d2h(void *dst, const void *src, size_t bytes) { tq_d2h(dst, src, bytes); }
void tq_cxx_dev_zero(void *dst, size_t bytes) { tq_dev_zero(dst, bytes); }
