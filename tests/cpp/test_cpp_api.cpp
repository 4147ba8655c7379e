// Exercises the C++ host layer (libmolgrid_b200/cpp/include/libmolgrid) on a GPU.
// usage: test_cpp_api <input.bin> <output.bin>
// The input holds seeded arrays written by tests/test_cpp_api_gpu.py, which also checks the arrays
// this program writes against the CPU oracle.  Structural checks (exceptions, MGrid behaviour) are
// asserted here and reported through the exit code.
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

  std::fclose(out);
  std::fclose(in);
  std::printf(failures ? "%d checks FAILED\n" : "all checks passed\n", failures);
  return failures ? 1 : 0;
}
