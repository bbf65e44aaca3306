// Which earlier keys a query may read, shared by the attention kernels.
//
// A query at position p always reads key p and never a later one.  Of the earlier keys it reads
//   all of them                                   (window = 0, chunk = 0),
//   the last `window` positions, p included        (window > 0:  j > p - window),
//   those of its own block of `chunk` positions    (chunk > 0:   j / chunk == p / chunk; blocks are
//                                                   counted from position 0 of the request),
// and, whatever the rule, the first `keep` keys of the request (keep > 0: keys that stay visible
// after a window has moved past them; they keep their own positions).
//
// Kernels walk a query's keys as one run of *virtual* indices v in [vlo, p]: with lo the first key
// of the rule and nk = min(keep, lo) kept keys before it, vlo = lo - nk, and v stands for key
// v - vlo if v < lo, else for key v itself.  So the kept keys ride directly in front of the rule's
// range and a kernel's chunking of [vlo, p] needs no second loop.
#pragma once

struct AttnMask {
    int window;     // 0: none
    int chunk;      // 0: none
    int keep;       // 0: none
};

__host__ __device__ __forceinline__ int mask_lo(const AttnMask& m, int pos) {
    int lo = 0;
    if (m.window > 0) lo = pos - m.window + 1 > 0 ? pos - m.window + 1 : 0;
    if (m.chunk > 0) {
        const int c = pos - pos % m.chunk;
        lo = c > lo ? c : lo;
    }
    return lo;
}

// first virtual index of a query whose rule starts at lo
__host__ __device__ __forceinline__ int mask_vlo(const AttnMask& m, int lo) { return lo - (m.keep < lo ? m.keep : lo); }

// the key a virtual index stands for
__host__ __device__ __forceinline__ int mask_key(int v, int vlo, int lo) { return v < lo ? v - vlo : v; }

// whether the query at position p reads key j (j <= p is the caller's to check or to imply)
__host__ __device__ __forceinline__ bool mask_sees(const AttnMask& m, int p, int j) {
    return j <= p && (j >= mask_lo(m, p) || j < m.keep);
}
