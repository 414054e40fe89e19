// The handle behind hb_a2a_* (peer-memory exchange) and what a kernel of another file needs to
// place records into the owners' slabs itself instead of going through hb_a2a_push.
#pragma once

#include "common.cuh"

struct hb_a2a {
  int rank, world;
  int64_t cap;        // rows per source slab
  int64_t row_bytes;
  size_t area_bytes;
  char* local[2];            // this rank's receive areas
  char* peer[2][64];         // peer[p][r] = rank r's area of parity p in this process
  bool opened[64];
  // device copy of the destination pointers for the push kernel
  struct Dest {
    unsigned long long* flags[64];  // parity-0 area of every rank
    int64_t* counts[64];
    int64_t* ids[64];
    int64_t* cnt[64];
    char* rows[64];
  };
  Dest* dest_dev[2];
  unsigned long long* epoch_dev;  // number of fences done, on the device (graph replay safe)
  int parity;  // parity of the NEXT push
};

namespace hb {

// A sender that places its records itself: record k for owner c goes to index rank * cap + k of
// dest->ids[c] / dest->cnt[c] (k < cap).  a2a_direct_begin hands out the destination table of the
// next push and its parity (like hb_a2a_push, the areas alternate); a2a_direct_publish, after the
// kernel that stored the records, tells every owner how many it got (counts_dev[c], clamped to cap).
int a2a_direct_begin(hb_a2a* a, const hb_a2a::Dest** dest, int* parity);
int a2a_direct_publish(hb_a2a* a, int parity, const unsigned long long* counts_dev, cudaStream_t st);

}  // namespace hb
