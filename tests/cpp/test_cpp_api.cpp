// Exercises the C++ host layer (libmolgrid_b200/cpp/include/libmolgrid) on a GPU.
// usage: test_cpp_api <input.bin> <output.bin>
// The input holds seeded arrays written by tests/test_cpp_api_gpu.py, which also checks the arrays
// this program writes against the CPU oracle.  Structural checks (exceptions, MGrid behaviour) are
// asserted here and reported through the exit code.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "libmolgrid/libmolgrid.h"

using namespace libmolgrid;

static int failures = 0;
#define EXPECT(cond)                                                     \
  do {                                                                   \
    if (!(cond)) { std::printf("FAILED %s:%d %s\n", __FILE__, __LINE__, #cond); failures++; } \
  } while (0)
#define EXPECT_THROW(stmt, type)                     \
  do {                                               \
    bool caught = false;                             \
    try { stmt; } catch (const type&) { caught = true; } catch (...) {} \
    if (!caught) { std::printf("FAILED %s:%d expected " #type "\n", __FILE__, __LINE__); failures++; } \
  } while (0)

static std::vector<float> read_floats(FILE* f, size_t n) {
  std::vector<float> v(n);
  if (n && std::fread(v.data(), sizeof(float), n, f) != n) { std::printf("short input\n"); std::exit(2); }
  return v;
}
static void write_grid(FILE* f, const MGrid4f& g) {
  Grid4f c = g.cpu();
  std::fwrite(c.data(), sizeof(float), c.size(), f);
}
template <class G>
static void write_any(FILE* f, const G& g) {
  auto c = g.cpu();
  std::fwrite(c.data(), sizeof(float), c.size(), f);
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  FILE* in = std::fopen(argv[1], "rb");
  FILE* out = std::fopen(argv[2], "wb");
  if (!in || !out) return 2;
  int hdr[4];
  if (std::fread(hdr, sizeof(int), 4, in) != 4) return 2;
  const int N = hdr[0], T = hdr[1], NL = hdr[2], K = hdr[3];  // receptor atoms, types, ligand atoms, interp channels
  std::vector<float> coords = read_floats(in, N * 3), types = read_floats(in, N), radii = read_floats(in, N);
  std::vector<float> lcoords = read_floats(in, NL * 3), ltypes = read_floats(in, NL), lradii = read_floats(in, NL);
  std::vector<float> tr = read_floats(in, 10);

  GridMaker gm(0.5, 11.5);
  EXPECT(gm.get_first_dim() == 24);
  const unsigned D = gm.get_first_dim();
  std::vector<float> diffv = read_floats(in, (size_t)T * D * D * D);
  std::vector<float> ingrid = read_floats(in, (size_t)K * D * D * D);
  float3 center = make_float3(0.1f, -0.2f, 0.3f);

  // ---- 1. index forward on device views of managed grids
  MGrid2f mc(N, 3); MGrid1f mt(N), mr(N);
  std::memcpy(mc.cpu().data(), coords.data(), coords.size() * 4);
  std::memcpy(mt.cpu().data(), types.data(), types.size() * 4);
  std::memcpy(mr.cpu().data(), radii.data(), radii.size() * 4);
  MGrid4f grid(T, D, D, D);
  {
    Grid4fCUDA g = grid.gpu();
    gm.forward(center, mc.gpu(), mt.gpu(), mr.gpu(), g);
    gm.check_types();
  }
  EXPECT(grid.ongpu());
  write_grid(out, grid);

  // ---- 2. the host-grid overload gives the same grid
  {
    MGrid4f hostgrid(T, D, D, D);
    Grid4f hg = hostgrid.cpu();
    Grid2f hc(coords.data(), N, 3); Grid1f ht(types.data(), N), hr(radii.data(), N);
    gm.forward(center, hc, ht, hr, hg);
    Grid4f a = grid.cpu();
    // the order in which a voxel's atoms are summed is not fixed between launches, so two runs
    // agree to rounding, not bit for bit
    bool same = true;
    for (size_t i = 0; i < a.size(); i++) {
      float d = a.data()[i] - hg.data()[i];
      same = same && (d < 0 ? -d : d) <= 1e-6f + 1e-5f * a.data()[i];
    }
    EXPECT(same);
  }

  // ---- 3. backward
  MGrid4f diff(T, D, D, D);
  std::memcpy(diff.cpu().data(), diffv.data(), diffv.size() * 4);
  MGrid2f ag(N, 3);
  {
    Grid2fCUDA g = ag.gpu();
    gm.backward(center, mc.gpu(), mt.gpu(), mr.gpu(), diff.gpu(), g);
  }
  write_any(out, ag);

  // ---- 4. Example of two coordinate sets under a Transform (fused into the gridding kernels)
  std::vector<float3> rc, lc;
  for (int i = 0; i < N; i++) rc.push_back(make_float3(coords[3 * i], coords[3 * i + 1], coords[3 * i + 2]));
  for (int i = 0; i < NL; i++) lc.push_back(make_float3(lcoords[3 * i], lcoords[3 * i + 1], lcoords[3 * i + 2]));
  Example ex;
  ex.sets.push_back(CoordinateSet(rc, types, radii, T));
  ex.sets.push_back(CoordinateSet(lc, ltypes, lradii, T));
  EXPECT(ex.num_coordinates() == (size_t)(N + NL));
  CoordinateSet merged = ex.merge_coordinates();
  EXPECT(merged.max_type == (unsigned)(2 * T) && merged.size() == (unsigned)(N + NL));
  Transform t(Quaternion(tr[0], tr[1], tr[2], tr[3]), make_float3(tr[4], tr[5], tr[6]), make_float3(tr[7], tr[8], tr[9]));
  MGrid4f exgrid(2 * T, D, D, D);
  {
    Grid4fCUDA g = exgrid.gpu();
    gm.forward(ex, t, g);
  }
  write_grid(out, exgrid);
  {
    MGrid4f wrong(T, D, D, D);
    Grid4fCUDA g = wrong.gpu();
    EXPECT_THROW(gm.forward(ex, t, g), std::out_of_range);  // channel count of the merged example
  }

  // ---- 5. vector<Example> in one batched pass, default centre = centre of the last set
  std::vector<Example> batch = {ex, ex};
  batch[1].sets[1] = CoordinateSet(rc, types, radii, T);  // different second example
  MGrid5f bgrid(2, 2 * T, D, D, D);
  {
    Grid5fCUDA g = bgrid.gpu();
    gm.forward(batch, g);
  }
  write_any(out, bgrid);
  float3 c0 = ex.sets.back().center();
  std::fwrite(&c0, sizeof(float), 3, out);

  // ---- 6. transform of coordinates and quaternion arithmetic on the host
  MGrid2f moved(N, 3);
  {
    Grid2fCUDA g = moved.gpu();
    t.forward(mc.gpu(), g);
  }
  write_any(out, moved);
  {
    Quaternion a(tr[0], tr[1], tr[2], tr[3]), b(0.5f, -0.25f, 0.75f, 1.5f);
    Quaternion p = a * b, q = a / b, inv = a.inverse();
    float3 r = a.rotate(coords[0], coords[1], coords[2]);
    float v[15] = {p.R_component_1(), p.R_component_2(), p.R_component_3(), p.R_component_4(),
                   q.R_component_1(), q.R_component_2(), q.R_component_3(), q.R_component_4(),
                   inv.R_component_1(), inv.R_component_2(), inv.R_component_3(), inv.R_component_4(), r.x, r.y, r.z};
    std::fwrite(v, sizeof(float), 15, out);
  }

  // ---- 7. interpolation
  GridInterpolater gi(0.5, 11.5, 0.5, 11.5);
  MGrid4f src(K, D, D, D), dst(K, D, D, D);
  std::memcpy(src.cpu().data(), ingrid.data(), ingrid.size() * 4);
  {
    Grid4fCUDA g = dst.gpu();
    gi.forward(src.gpu(), t, g);
    Grid4fCUDA same = src.gpu();
    EXPECT_THROW(gi.forward(same, t, same), std::invalid_argument);
  }
  write_grid(out, dst);
  {
    // host grids, and the overload that draws its own transform (identity when nothing is random)
    std::vector<float> hout(ingrid.size(), -1.f), hout2(ingrid.size(), -1.f);
    Grid4f hin(ingrid.data(), K, D, D, D), ho(hout.data(), K, D, D, D), ho2(hout2.data(), K, D, D, D);
    gi.forward(hin, t, ho);
    Grid4f hd = dst.cpu();
    bool same = true;
    for (size_t i = 0; i < hout.size(); i++) same = same && hout[i] == hd.data()[i];
    EXPECT(same);
    gi.forward(hin, ho2);
    same = true;
    for (size_t i = 0; i < hout2.size(); i++) same = same && hout2[i] == ingrid[i];
    EXPECT(same);
  }
  {
    // backward is the adjoint of forward: <forward(src), dst> == <src, backward(dst)>
    MGrid4f back(K, D, D, D);
    Grid4fCUDA gb = back.gpu();
    gi.backward(dst.gpu(), t, gb);
    double lhs = 0, rhs = 0;
    Grid4f hs = src.cpu(), hd = dst.cpu(), hb = back.cpu();
    for (size_t i = 0; i < hs.size(); i++) {
      lhs += (double)hd.data()[i] * hd.data()[i];
      rhs += (double)hs.data()[i] * hb.data()[i];
    }
    EXPECT(lhs > 1.0 && std::fabs(lhs - rhs) <= 1e-4 * lhs);
  }

  // ---- 8. argument errors carry the reference's exception types
  {
    MGrid4f bad(T, D + 1, D, D);
    Grid4fCUDA g = bad.gpu();
    EXPECT_THROW(gm.forward(center, mc.gpu(), mt.gpu(), mr.gpu(), g), std::out_of_range);
    MGrid1f shortr(N - 1);
    Grid4fCUDA g2 = grid.gpu();
    EXPECT_THROW(gm.forward(center, mc.gpu(), mt.gpu(), shortr.gpu(), g2), std::out_of_range);
    Grid2fCUDA agv = ag.gpu();
    EXPECT_THROW(gm.backward(center, mc.gpu(), mt.gpu(), shortr.gpu(), diff.gpu(), agv), std::invalid_argument);
    GridMaker rti(0.5, 11.5, false, true);
    EXPECT_THROW(rti.backward(center, mc.gpu(), mt.gpu(), mr.gpu(), diff.gpu(), agv), std::invalid_argument);
    MGrid1f bigt(N);
    for (int i = 0; i < N; i++) bigt(i) = (float)T;   // one past the last channel
    gm.forward(center, mc.gpu(), bigt.gpu(), mr.gpu(), g2);
    EXPECT_THROW(gm.check_types(), std::out_of_range);
  }

  {
    // double grids keep their signatures and throw
    MGrid4d dgrid(T, D, D, D);
    Grid4dCUDA dg = dgrid.gpu();
    EXPECT_THROW(gm.forward(center, mc.gpu(), mt.gpu(), mr.gpu(), dg), std::invalid_argument);
  }

  // ---- 10. host-grid overloads of the backward passes agree with the device overloads
  {
    auto close = [](const float* a, const float* b, size_t n, float scale) {
      for (size_t i = 0; i < n; i++) {
        float d = a[i] - b[i];
        if ((d < 0 ? -d : d) > 1e-5f * scale + 1e-4f * (a[i] < 0 ? -a[i] : a[i])) return false;
      }
      return true;
    };
    Grid2f hc(coords.data(), N, 3); Grid1f ht(types.data(), N), hr(radii.data(), N);
    Grid4f hd(diffv.data(), T, D, D, D);
    std::vector<float> hagv(N * 3, -1.f);
    Grid2f hag(hagv.data(), N, 3);
    gm.backward(center, hc, ht, hr, hd, hag);
    EXPECT(close(hagv.data(), ag.cpu().data(), hagv.size(), 10.f));

    // index-typed coordinate set, host grids: forward, backward, relevance
    CoordinateSet cs(rc, types, radii, T);
    MGrid4f csgrid(T, D, D, D);
    Grid4f csg = csgrid.cpu();
    gm.forward(center, cs, csg);
    {
      Grid4fCUDA g = grid.gpu();   // section 8 left another case in it
      gm.forward(center, mc.gpu(), mt.gpu(), mr.gpu(), g);
    }
    EXPECT(close(csg.data(), grid.cpu().data(), csg.size(), 1.f));
    std::vector<float> hag2(N * 3, -1.f);
    Grid2f hag2g(hag2.data(), N, 3);
    gm.backward(center, cs, hd, hag2g);
    EXPECT(close(hag2.data(), hagv.data(), hag2.size(), 10.f));
    std::vector<float> relh(N, -1.f);
    Grid1f relhg(relh.data(), N);
    gm.backward_relevance(center, cs, csg, hd, relhg);
    MGrid1f reld(N);
    {
      Grid1fCUDA g = reld.gpu();
      gm.backward_relevance(center, mc.gpu(), mt.gpu(), mr.gpu(), grid.gpu(), diff.gpu(), g);
    }
    EXPECT(close(relh.data(), reld.cpu().data(), relh.size(), 10.f));

    // vector types: host and device overloads of backward and backward_gradients, arrays and sets
    std::vector<float> tv((size_t)N * T, 0.f);
    for (int i = 0; i < N; i++) {
      tv[(size_t)i * T + ((int)types[i] % T + T) % T] = 0.75f;
      tv[(size_t)i * T + (i % T)] += 0.25f;
    }
    Grid2f htv(tv.data(), N, T);
    std::vector<float> vag(N * 3), vtg((size_t)N * T);
    Grid2f vagg(vag.data(), N, 3), vtgg(vtg.data(), N, T);
    gm.backward(center, hc, htv, hr, hd, vagg, vtgg);
    MGrid2f mtv(N, T), dag(N, 3), dtg(N, T);
    std::memcpy(mtv.cpu().data(), tv.data(), tv.size() * 4);
    {
      Grid2fCUDA a = dag.gpu(), b = dtg.gpu();
      gm.backward(center, mc.gpu(), mtv.gpu(), mr.gpu(), diff.gpu(), a, b);
    }
    EXPECT(close(vag.data(), dag.cpu().data(), vag.size(), 10.f));
    EXPECT(close(vtg.data(), dtg.cpu().data(), vtg.size(), 10.f));
    CoordinateSet vs(hc, htv, hr);
    EXPECT(vs.has_vector_types() && vs.num_types() == (unsigned)T);
    std::vector<float> sag(N * 3), stg((size_t)N * T);
    Grid2f sagg(sag.data(), N, 3), stgg(stg.data(), N, T);
    gm.backward(center, vs, hd, sagg, stgg);
    EXPECT(close(sag.data(), vag.data(), sag.size(), 10.f));
    EXPECT_THROW(gm.backward(center, cs, hd, sagg, stgg), std::invalid_argument);   // no vector types

    std::vector<float> ddh((size_t)T * D * D * D), addh(N * 3), tddh((size_t)N * T, 1.f);
    Grid4f ddhg(ddh.data(), T, D, D, D);
    Grid2f addhg(addh.data(), N, 3), tddhg(tddh.data(), N, T);
    gm.backward_gradients(center, hc, htv, hr, hd, vagg, vtgg, ddhg, addhg, tddhg);
    MGrid4f ddd(T, D, D, D);
    MGrid2f addd(N, 3), tddd(N, T);
    {
      Grid4fCUDA a = ddd.gpu();
      Grid2fCUDA b = addd.gpu(), c = tddd.gpu();
      gm.backward_gradients(center, vs, diff.gpu(), dag.gpu(), dtg.gpu(), a, b, c);
    }
    EXPECT(close(ddh.data(), ddd.cpu().data(), ddh.size(), 100.f));
    EXPECT(close(addh.data(), addd.cpu().data(), addh.size(), 1000.f));
    bool zero = true;
    for (float v : tddh) zero = zero && v == 0.f;
    EXPECT(zero);   // the reference leaves type_diffdiff at zero
  }

  // ---- 9. managed grids: shared storage, slices, clone, resize
  {
    MGrid2f m(3, 4);
    m(1, 2) = 5.f;
    MGrid1f row = m[1];
    EXPECT(row(2) == 5.f);
    row(3) = 7.f;
    EXPECT(m(1, 3) == 7.f);
    MGrid2f copy = m;          // shares storage
    MGrid2f deep = m.clone();  // does not
    m(0, 0) = 1.f;
    EXPECT(copy(0, 0) == 1.f && deep(0, 0) == 0.f);
    Grid2fCUDA g = m.gpu();
    EXPECT(m.ongpu() && copy.ongpu() && g.dimension(1) == 4);
    EXPECT(m(1, 2) == 5.f && m.oncpu());   // element access brings it back
    MGrid2f bigger = m.resized(5, 4);
    EXPECT(bigger.dimension(0) == 5 && bigger(1, 3) == 7.f && bigger(4, 3) == 0.f);
    EXPECT_THROW(m[3], std::out_of_range);
    Grid2f v = m.cpu();
    EXPECT(v[1][2] == 5.f && v(1, 3) == 7.f && v.offset(0) == 4 && v.size() == 12);
  }

  // ---- 10. batched arrays with per-example transforms and ragged atom counts (additions of this
  // library): the batch equals the examples gridded one by one; batched backward likewise, bit for bit
  {
    const int B = 2, NB = N;                 // example 1 uses only the first NL atoms of the padded row
    MGrid3f bc(B, NB, 3);
    MGrid2f bt(B, NB), br(B, NB), cen(B, 3), trs(B, 10);
    for (int b = 0; b < B; b++) {
      int n = b == 0 ? N : NL;
      const std::vector<float>& cs = b == 0 ? coords : lcoords;
      const std::vector<float>& ts = b == 0 ? types : ltypes;
      const std::vector<float>& rs = b == 0 ? radii : lradii;
      for (int i = 0; i < n; i++) {
        for (int k = 0; k < 3; k++) bc(b, i, k) = cs[i * 3 + k];
        bt(b, i) = ts[i];
        br(b, i) = rs[i];
      }
      for (int k = 0; k < 10; k++) trs(b, k) = tr[k];
      trs(b, 7) += 0.25f * b;                // a different translation per example
      for (int k = 0; k < 3; k++) cen(b, k) = tr[4 + k];
    }
    int counts_h[B] = {N, NL};
    int* counts = nullptr;
    EXPECT(cudaMalloc(&counts, sizeof counts_h) == cudaSuccess);
    EXPECT(cudaMemcpy(counts, counts_h, sizeof counts_h, cudaMemcpyHostToDevice) == cudaSuccess);
    MGrid5f outb(B, T, D, D, D);
    {
      Grid5fCUDA og = outb.gpu();
      gm.forward<2>(cen.gpu(), bc.gpu(), bt.gpu(), br.gpu(), og,
                    reinterpret_cast<const lmg_transform*>(trs.gpu().data()), counts);
    }
    MGrid5f diffb(B, T, D, D, D);
    for (int b = 0; b < B; b++)
      for (size_t i = 0; i < diffv.size(); i++) diffb.cpu().data()[b * diffv.size() + i] = diffv[i] * (b + 1);
    MGrid3f agb(B, NB, 3);
    {
      Grid3fCUDA ag = agb.gpu();
      gm.backward<2>(cen.gpu(), bc.gpu(), bt.gpu(), br.gpu(), diffb.gpu(), ag, nullptr,
                     reinterpret_cast<const lmg_transform*>(trs.gpu().data()), counts);
    }
    for (int b = 0; b < B; b++) {
      int n = b == 0 ? N : NL;
      MGrid2f c1(n, 3), ag1(n, 3);
      MGrid1f t1(n), r1(n);
      for (int i = 0; i < n; i++) {
        for (int k = 0; k < 3; k++) c1(i, k) = bc(b, i, k);
        t1(i) = bt(b, i);
        r1(i) = br(b, i);
      }
      Transform one(Quaternion(tr[0], tr[1], tr[2], tr[3]), make_float3(tr[4], tr[5], tr[6]),
                    make_float3(tr[7] + 0.25f * b, tr[8], tr[9]));
      MGrid4f o1(T, D, D, D), d1(T, D, D, D);
      for (size_t i = 0; i < diffv.size(); i++) d1.cpu().data()[i] = diffv[i] * (b + 1);
      {
        Grid4fCUDA og = o1.gpu();
        Grid2fCUDA ag = ag1.gpu();
        gm.forward(one.get_rotation_center(), c1.gpu(), t1.gpu(), r1.gpu(), og, &one);
        gm.backward(one.get_rotation_center(), c1.gpu(), t1.gpu(), r1.gpu(), d1.gpu(), ag, &one);
      }
      const float* want = o1.cpu().data();
      const float* got = outb.cpu().data() + (size_t)b * T * D * D * D;
      bool same = true, any = false;
      for (size_t i = 0; i < (size_t)T * D * D * D; i++) {
        same = same && std::fabs(got[i] - want[i]) <= 1e-6f + 1e-5f * std::fabs(want[i]);
        any = any || want[i] != 0.f;
      }
      EXPECT(same && any);
      bool equal = true;
      for (int i = 0; i < n; i++)
        for (int k = 0; k < 3; k++) equal = equal && agb(b, i, k) == ag1(i, k);
      EXPECT(equal);                          // the backward kernels sum in a fixed order
      for (int i = n; i < NB; i++) EXPECT(agb(b, i, 0) == 0.f && agb(b, i, 1) == 0.f && agb(b, i, 2) == 0.f);
    }
    cudaFree(counts);
  }

  // ---- 11. merge_coordinates: vector types win when every non-empty set has them
  {
    std::vector<float3> c2 = {make_float3(0, 0, 0), make_float3(1, 0, 0)};
    std::vector<std::vector<float>> v3 = {{1, 0, 0}, {0, 0.5f, 0.5f}}, v2 = {{0, 1}, {1, 0}};
    Example ex;
    ex.sets.push_back(CoordinateSet(c2, v3, std::vector<float>{1.f, 2.f, 3.f}));
    CoordinateSet empty;
    empty.max_type = 4;
    ex.sets.push_back(empty);
    ex.sets.push_back(CoordinateSet(c2, v2, std::vector<float>{4.f, 5.f}));
    CoordinateSet m = ex.merge_coordinates();
    EXPECT(m.has_vector_types() && m.size() == 4 && m.max_type == 9);
    EXPECT(m.type_vector.dimension(1) == 9 && m.radii.size() == 5);
    EXPECT(m.type_vector(1, 2) == 0.5f && m.type_vector(2, 8) == 1.f && m.type_vector(3, 7) == 1.f);
    EXPECT(m.type_vector(2, 0) == 0.f && m.radii(3) == 4.f);
    Example mixed;
    mixed.sets.push_back(CoordinateSet(c2, std::vector<float>{0.f, 1.f}, std::vector<float>{1.f, 1.f}, 2));
    mixed.sets.push_back(CoordinateSet(c2, v2, std::vector<float>{4.f, 5.f}));
    EXPECT_THROW(mixed.merge_coordinates(), std::invalid_argument);
  }

  std::fclose(out);
  std::fclose(in);
  std::printf(failures ? "%d checks FAILED\n" : "all checks passed\n", failures);
  return failures ? 1 : 0;
}
