// Selection order of a CPU top-k, reproduced for device code.
//
// The bank update picks its candidates with torch.topk on the CPU tensor of write
// gates (upstream src/coda_gqa_l/memory_banks.py:491,532,541: largest, unsorted)
// and ranks LRU victims with torch.topk on int64 stamps (memory_banks.py:663:
// smallest, sorted).  Which of several equal elements is returned, and in what
// order, is decided by the selection algorithm ATen runs on the host: a queue of
// (value, index) pairs that is either heap-selected (when k*64 <= n) or
// nth_element-partitioned and, for sorted=True, has its first k-1 entries sorted.
// With the default zero-initialised gate projection every gate is equal, so the
// whole candidate list is a tie-break.  The routines below restate those published
// algorithms (median-of-3 introselect with a final insertion sort, binary-heap
// select + sort-heap, introsort with a 16-element insertion-sort threshold) so that
// the device produces the same index lists; tests fuzz them against torch.topk.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TK_HD __host__ __device__ __forceinline__
#else
#define TK_HD inline
#endif

namespace topk_order {

template <typename V> struct Item { V v; int32_t i; };

// "a goes before b": largest-first for gates (NaN counts as largest), smallest-first for stamps.
template <typename V, bool LARGEST> struct Before {
  TK_HD bool operator()(const Item<V>& a, const Item<V>& b) const {
    if (LARGEST) return ((a.v != a.v) && !(b.v != b.v)) || (a.v > b.v);
    return (!(a.v != a.v) && (b.v != b.v)) || (a.v < b.v);
  }
};

template <typename It> TK_HD void swap_items(It* q, int a, int b) { It t = q[a]; q[a] = q[b]; q[b] = t; }

TK_HD int floor_log2(int n) { int r = 0; while (n > 1) { n >>= 1; ++r; } return r; }

template <typename It, typename Cmp>
TK_HD void median_to_first(It* q, int r, int a, int b, int c, Cmp before) {
  if (before(q[a], q[b])) {
    if (before(q[b], q[c])) swap_items(q, r, b);
    else if (before(q[a], q[c])) swap_items(q, r, c);
    else swap_items(q, r, a);
  } else if (before(q[a], q[c])) swap_items(q, r, a);
  else if (before(q[b], q[c])) swap_items(q, r, c);
  else swap_items(q, r, b);
}

// Hoare-style partition of [first,last) around the pivot stored at q[pivot]; no bounds guards
// are needed because the median-of-3 step leaves sentinels on both sides.
template <typename It, typename Cmp>
TK_HD int partition_unguarded(It* q, int first, int last, int pivot, Cmp before) {
  for (;;) {
    while (before(q[first], q[pivot])) ++first;
    --last;
    while (before(q[pivot], q[last])) --last;
    if (!(first < last)) return first;
    swap_items(q, first, last);
    ++first;
  }
}

template <typename It, typename Cmp>
TK_HD int partition_pivot(It* q, int first, int last, Cmp before) {
  int mid = first + (last - first) / 2;
  median_to_first(q, first, first + 1, mid, last - 1, before);
  return partition_unguarded(q, first + 1, last, first, before);
}

template <typename It, typename Cmp>
TK_HD void linear_insert_unguarded(It* q, int last, Cmp before) {
  It val = q[last];
  int next = last - 1;
  while (before(val, q[next])) { q[last] = q[next]; last = next; --next; }
  q[last] = val;
}

template <typename It, typename Cmp>
TK_HD void insertion_sort(It* q, int first, int last, Cmp before) {
  if (first == last) return;
  for (int i = first + 1; i != last; ++i) {
    if (before(q[i], q[first])) {
      It val = q[i];
      for (int j = i; j > first; --j) q[j] = q[j - 1];
      q[first] = val;
    } else {
      linear_insert_unguarded(q, i, before);
    }
  }
}

template <typename It, typename Cmp>
TK_HD void sift_up(It* q, int first, int hole, int top, It value, Cmp before) {
  int parent = (hole - 1) / 2;
  while (hole > top && before(q[first + parent], value)) {
    q[first + hole] = q[first + parent];
    hole = parent;
    parent = (hole - 1) / 2;
  }
  q[first + hole] = value;
}

template <typename It, typename Cmp>
TK_HD void sift_down(It* q, int first, int hole, int len, It value, Cmp before) {
  const int top = hole;
  int child = hole;
  while (child < (len - 1) / 2) {
    child = 2 * (child + 1);
    if (before(q[first + child], q[first + child - 1])) --child;
    q[first + hole] = q[first + child];
    hole = child;
  }
  if ((len & 1) == 0 && child == (len - 2) / 2) {
    child = 2 * (child + 1);
    q[first + hole] = q[first + child - 1];
    hole = child - 1;
  }
  sift_up(q, first, hole, top, value, before);
}

template <typename It, typename Cmp>
TK_HD void build_heap(It* q, int first, int last, Cmp before) {
  int len = last - first;
  if (len < 2) return;
  for (int parent = (len - 2) / 2;; --parent) {
    sift_down(q, first, parent, len, q[first + parent], before);
    if (parent == 0) return;
  }
}

template <typename It, typename Cmp>
TK_HD void pop_to(It* q, int first, int last, int result, Cmp before) {
  It value = q[result];
  q[result] = q[first];
  sift_down(q, first, 0, last - first, value, before);
}

template <typename It, typename Cmp>
TK_HD void heap_select(It* q, int first, int middle, int last, Cmp before) {
  build_heap(q, first, middle, before);
  for (int i = middle; i < last; ++i)
    if (before(q[i], q[first])) pop_to(q, first, middle, i, before);
}

template <typename It, typename Cmp>
TK_HD void heap_sort_range(It* q, int first, int last, Cmp before) {
  while (last - first > 1) { --last; pop_to(q, first, last, last, before); }
}

template <typename It, typename Cmp>
TK_HD void select_nth(It* q, int first, int nth, int last, Cmp before) {
  if (first == last || nth == last) return;
  int depth = floor_log2(last - first) * 2;
  while (last - first > 3) {
    if (depth == 0) {
      heap_select(q, first, nth + 1, last, before);
      swap_items(q, first, nth);
      return;
    }
    --depth;
    int cut = partition_pivot(q, first, last, before);
    if (cut <= nth) first = cut; else last = cut;
  }
  insertion_sort(q, first, last, before);
}

// Introsort of [first,last): quicksort partitions down to 16-element runs, heap sort when the
// depth budget (2*floor(log2 n)) runs out, then one insertion-sort pass over the whole range.
// The recursion of the textbook form is replaced by an explicit stack of pending right-hand
// parts; the parts are disjoint, so the order in which they are processed does not change
// the result, only the per-part depth budget does, and that is carried on the stack.
template <typename It, typename Cmp>
TK_HD void sort_range(It* q, int first, int last, Cmp before) {
  if (first == last) return;
  int s_lo[64], s_hi[64], s_depth[64];
  int sp = 0;
  s_lo[0] = first; s_hi[0] = last; s_depth[0] = floor_log2(last - first) * 2; sp = 1;
  while (sp > 0) {
    --sp;
    int lo = s_lo[sp], hi = s_hi[sp], depth = s_depth[sp];
    while (hi - lo > 16) {
      if (depth == 0) {
        build_heap(q, lo, hi, before);
        heap_sort_range(q, lo, hi, before);
        break;
      }
      --depth;
      int cut = partition_pivot(q, lo, hi, before);
      s_lo[sp] = cut; s_hi[sp] = hi; s_depth[sp] = depth; ++sp;
      hi = cut;
    }
  }
  if (last - first > 16) {
    insertion_sort(q, first, first + 16, before);
    for (int i = first + 16; i != last; ++i) linear_insert_unguarded(q, i, before);
  } else {
    insertion_sort(q, first, last, before);
  }
}

// Fill q[0..n) with (value, index) pairs beforehand.  Afterwards q[0..k) holds the selection
// in the order the host top-k returns it.
template <typename V, bool LARGEST>
TK_HD void topk_queue(Item<V>* q, int n, int k, bool sorted) {
  if (k <= 0 || n <= 0) return;
  Before<V, LARGEST> before;
  if ((int64_t)k * 64 <= (int64_t)n) {
    heap_select(q, 0, k, n, before);
    heap_sort_range(q, 0, k, before);
  } else {
    select_nth(q, 0, k - 1, n, before);
    if (sorted) sort_range(q, 0, k - 1, before);
  }
}

}  // namespace topk_order
