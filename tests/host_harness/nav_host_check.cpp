// TEST HARNESS ONLY.  Compiles the per-thread query functions of
// bps_nav_b200/csrc/nav_query.cuh with the host C++ compiler so the index
// arithmetic and control flow can be checked against the reference library
// on a machine without a GPU.  The shipped library never links this file and
// has no CPU execution path.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../bps_nav_b200/csrc/nav_query.cuh"
#include "../../bps_nav_b200/csrc/navmesh_host.h"

using namespace bpsn;

struct HChk {
  HostScene hs;
  NavScene sc;
  AStarScratch* scratch;
};

extern "C" {

void* hchk_load(const char* path, char* err, int errlen) {
  FILE* fp = fopen(path, "rb");
  if (!fp) {
    snprintf(err, errlen, "cannot open %s", path);
    return nullptr;
  }
  std::vector<uint8_t> buf;
  fseek(fp, 0, SEEK_END);
  long n = ftell(fp);
  fseek(fp, 0, SEEK_SET);
  buf.resize(n);
  if (fread(buf.data(), 1, n, fp) != static_cast<size_t>(n)) {
    fclose(fp);
    snprintf(err, errlen, "short read");
    return nullptr;
  }
  fclose(fp);
  HChk* h = new HChk();
  std::string e = parseNavmesh(buf.data(), buf.size(), &h->hs);
  if (!e.empty()) {
    snprintf(err, errlen, "%s", e.c_str());
    delete h;
    return nullptr;
  }
  h->sc = h->hs.view();
  h->scratch = new AStarScratch();
  return h;
}

void hchk_free(void* p) {
  HChk* h = static_cast<HChk*>(p);
  delete h->scratch;
  delete h;
}

void hchk_info(void* p, int* out) {
  HChk* h = static_cast<HChk*>(p);
  out[0] = h->sc.npolys;
  out[1] = h->sc.nverts;
  out[2] = h->sc.nbv;
  out[3] = h->hs.numDisabled;
  out[4] = h->hs.numIslands;
  out[5] = static_cast<int>(h->sc.refBase);
}

void hchk_snap_batch(void* p, int n, const float* pts, float* out_xyz, uint32_t* out_ref) {
  HChk* h = static_cast<HChk*>(p);
  for (int i = 0; i < n; ++i)
    snapPoint(h->sc, pts + 3 * i, out_xyz + 3 * i, out_ref + i);
}

void hchk_try_step_batch(void* p, int n, const float* start, const uint32_t* start_ref,
                         const float* end, float* out_xyz, uint32_t* out_ref) {
  HChk* h = static_cast<HChk*>(p);
  for (int i = 0; i < n; ++i) {
    float pos[3] = {start[3 * i], start[3 * i + 1], start[3 * i + 2]};
    uint32_t ref = start_ref[i];
    tryStep(h->sc, pos, &ref, end + 3 * i);
    out_xyz[3 * i] = pos[0];
    out_xyz[3 * i + 1] = pos[1];
    out_xyz[3 * i + 2] = pos[2];
    out_ref[i] = ref;
  }
}

void hchk_geodesic_batch(void* p, int n, const float* s, const uint32_t* sref, const float* e,
                         const uint32_t* eref, float* out, uint32_t* status) {
  HChk* h = static_cast<HChk*>(p);
  for (int i = 0; i < n; ++i) {
    uint32_t st = 0;
    out[i] = geodesic(h->sc, h->scratch, s + 3 * i, sref[i], e + 3 * i, eref[i], &st);
    status[i] = st;
  }
}

#if defined(BPSN_QUERY_STATS)
long hchk_pops() { return bpsn::g_statPops; }
#endif

}  // extern "C"
