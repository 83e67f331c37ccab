/* The cache manager's C functions (cache_core.cpp): page pools with a FIFO free list, request
 * slots and a block table per request and cache group.  Host bookkeeping only. */
#ifndef KIPP_CACHE_CORE_H
#define KIPP_CACHE_CORE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define KIPP_CM_OK 0
#define KIPP_CM_OUT_OF_PAGES (-1)
#define KIPP_CM_OUT_OF_SLOTS (-2)
#define KIPP_CM_ARGUMENT (-3)
#define KIPP_CM_BEHIND_WINDOW (-4)
#define KIPP_CM_CHECK (-5)
#define KIPP_CM_WINDOW_REFUSES (-8)

void* kipp_cm_create(int n_groups, const int* n_pages, const int* windows, int page_size, int max_requests);
void kipp_cm_destroy(void* h);
void* kipp_cm_pool(void* h, int group);
void* kipp_cm_slots(void* h);
int kipp_pool_free_pages(void* pool);
int kipp_slots_free_count(void* slots);
int kipp_cm_admit(void* h, int64_t rid);
int kipp_cm_release(void* h, int64_t rid);
int kipp_cm_slot(void* h, int64_t rid);
int kipp_cm_length(void* h, int64_t rid);
int kipp_cm_missing_pages(void* h, int64_t rid, int new_length, int* out);
int kipp_cm_reserve(void* h, int n, const int64_t* rids, const int* new_lengths);
int kipp_cm_advance(void* h, int64_t rid, int new_length);
int kipp_cm_truncate(void* h, int64_t rid, int new_length, int* refusing_group);
int kipp_cm_table_len(void* h, int64_t rid, int group);
int kipp_cm_table(void* h, int64_t rid, int group, int* out, int cap);
int kipp_cm_rows(void* h, int group, int n, const int64_t* rids, int width, int* out);
int kipp_cm_pages_held(void* h, int64_t rid, int* out);
int kipp_cm_check(void* h);
#ifdef __cplusplus
}
#endif
#endif
