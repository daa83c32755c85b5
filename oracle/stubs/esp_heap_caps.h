#pragma once
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#define MALLOC_CAP_DEFAULT (1 << 12)
#define MALLOC_CAP_INTERNAL (1 << 11)
#define MALLOC_CAP_SPIRAM (1 << 10)
#define MALLOC_CAP_8BIT (1 << 2)
#define MALLOC_CAP_SIMD (1 << 21)
#define MALLOC_CAP_TCM (1 << 15)
#define MALLOC_CAP_DMA (1 << 3)
#define HEAP_IRAM_ATTR
static inline void *heap_caps_aligned_alloc(size_t al, size_t n, uint32_t caps) { (void)caps; void *p = NULL; if (posix_memalign(&p, al < 16 ? 16 : al, n ? n : 16)) return NULL; return p; }
static inline void *heap_caps_aligned_calloc(size_t al, size_t n, size_t sz, uint32_t caps) { void *p = heap_caps_aligned_alloc(al, n * sz, caps); if (p) memset(p, 0, n * sz); return p; }
static inline void *heap_caps_malloc(size_t n, uint32_t caps) { return heap_caps_aligned_alloc(16, n, caps); }
static inline void *heap_caps_calloc(size_t n, size_t sz, uint32_t caps) { return heap_caps_aligned_calloc(16, n, sz, caps); }
static inline void heap_caps_free(void *p) { free(p); }
static inline size_t heap_caps_get_largest_free_block(uint32_t caps) { (void)caps; return (size_t)1 << 30; }
static inline size_t heap_caps_get_free_size(uint32_t caps) { (void)caps; return (size_t)1 << 30; }
static inline size_t heap_caps_get_total_size(uint32_t caps) { (void)caps; return (size_t)1 << 30; }
static inline size_t heap_caps_get_allocated_size(void *p) { (void)p; return 0; }
