// CoordinateSet and Example: the containers the GridMaker/Transform convenience overloads take
// (reference: include/libmolgrid/coordinateset.h, include/libmolgrid/example.h).  Only what feeds the
// gridding path is here: construction from arrays, type queries, center(), host/device residency,
// clone(), and Example::merge_coordinates.  Construction from OpenBabel molecules
// and the type-summing helpers are not part of this library.
#ifndef LMGB200_COORDINATESET_H_
#define LMGB200_COORDINATESET_H_

#include <vector>

#include "libmolgrid/managed_grid.h"

namespace libmolgrid {

struct CoordinateSet {
  MGrid2f coords{0, 3};
  MGrid1f type_index{0};
  MGrid2f type_vector{0, 0};
  MGrid1f radii{0};       // per atom, or per type when used with type-indexed radii
  unsigned max_type = 0;  // number of index types
  const char* src = nullptr;

  CoordinateSet() {}

  // index types
  CoordinateSet(const std::vector<float3>& c, const std::vector<float>& t, const std::vector<float>& r, unsigned maxt)
      : coords(c.size(), 3), type_index(c.size()), radii(c.size()), max_type(maxt) {
    if (t.size() != c.size() || r.size() != c.size())
      throw std::invalid_argument("Types/radii and coordinates are of different sizes");
    for (size_t i = 0; i < c.size(); i++) {
      coords(i, 0) = c[i].x; coords(i, 1) = c[i].y; coords(i, 2) = c[i].z;
      type_index(i) = t[i];
      radii(i) = r[i];
    }
  }
  CoordinateSet(const std::vector<float3>& c, const std::vector<int>& t, const std::vector<float>& r, unsigned maxt)
      : CoordinateSet(c, std::vector<float>(t.begin(), t.end()), r, maxt) {}

  template <bool G>
  CoordinateSet(const Grid<float, 2, G>& c, const Grid<float, 1, G>& t, const Grid<float, 1, G>& r, unsigned maxt)
      : coords(c.dimension(0), 3), type_index(t.size()), radii(r.size()), max_type(maxt) {
    if (c.dimension(1) != 3) throw std::invalid_argument("Coordinates have wrong secondary dimension");
    if (t.size() != c.dimension(0) || r.size() != c.dimension(0))
      throw std::invalid_argument("Types/radii and coordinates are of different sizes");
    coords.copyFrom(c); type_index.copyFrom(t); radii.copyFrom(r);
  }

  // vector types
  CoordinateSet(const std::vector<float3>& c, const std::vector<std::vector<float>>& t, const std::vector<float>& r)
      : coords(c.size(), 3), type_vector(c.size(), t.empty() ? 0 : t[0].size()), radii(r.size()),
        max_type(t.empty() ? 0 : (unsigned)t[0].size()) {
    if (t.size() != c.size()) throw std::invalid_argument("Types and coordinates are of different sizes");
    for (size_t i = 0; i < c.size(); i++) {
      coords(i, 0) = c[i].x; coords(i, 1) = c[i].y; coords(i, 2) = c[i].z;
      for (size_t k = 0; k < t[i].size(); k++) type_vector(i, k) = t[i][k];
    }
    for (size_t i = 0; i < r.size(); i++) radii(i) = r[i];
  }
  template <bool G>
  CoordinateSet(const Grid<float, 2, G>& c, const Grid<float, 2, G>& t, const Grid<float, 1, G>& r)
      : coords(c.dimension(0), 3), type_vector(t.dimension(0), t.dimension(1)), radii(r.size()),
        max_type((unsigned)t.dimension(1)) {
    if (c.dimension(1) != 3) throw std::invalid_argument("Coordinates have wrong secondary dimension");
    if (t.dimension(0) != c.dimension(0)) throw std::invalid_argument("Types and coordinates are of different sizes");
    coords.copyFrom(c); type_vector.copyFrom(t); radii.copyFrom(r);
  }

  // as in the reference, an empty set counts as having both kinds of types
  bool has_indexed_types() const { return type_index.size() > 0 || coords.size() == 0; }
  bool has_vector_types() const { return type_vector.size() > 0 || coords.size() == 0; }
  unsigned num_types() const { return max_type; }
  void set_num_types(unsigned m) { max_type = m; }
  unsigned size() const { return (unsigned)coords.dimension(0); }

  // mean coordinate, accumulated in single precision in atom order
  float3 center() const {
    float3 s = make_float3(0, 0, 0);
    unsigned n = size();
    if (n == 0) return s;
    Grid2f c = coords.cpu();
    for (unsigned i = 0; i < n; i++) { s.x += c(i, 0); s.y += c(i, 1); s.z += c(i, 2); }
    s.x /= n; s.y /= n; s.z /= n;
    return s;
  }

  void togpu(bool copy = true) { coords.togpu(copy); type_index.togpu(copy); type_vector.togpu(copy); radii.togpu(copy); }
  void tocpu(bool copy = true) { coords.tocpu(copy); type_index.tocpu(copy); type_vector.tocpu(copy); radii.tocpu(copy); }

  CoordinateSet clone() const {
    CoordinateSet r(*this);
    r.coords = coords.clone(); r.type_index = type_index.clone();
    r.type_vector = type_vector.clone(); r.radii = radii.clone();
    return r;
  }
};

struct Example {
  std::vector<CoordinateSet> sets;
  std::vector<float> labels;
  int group = -1;
  bool seqcont = false;

  size_t num_coordinates() const {
    size_t n = 0;
    for (const auto& s : sets) n += s.size();
    return n;
  }
  // total number of index types when every set keeps its own type range
  size_t num_types(bool unique_index_types = true) const {
    size_t total = 0, mx = 0;
    for (const auto& s : sets) { total += s.max_type; mx = std::max<size_t>(mx, s.max_type); }
    return unique_index_types ? total : mx;
  }

  // every non-empty set from `start` on has vector (index) types; empty sets count as both
  bool has_vector_types(unsigned start = 0) const {
    for (size_t i = start; i < sets.size(); i++)
      if (sets[i].size() > 0 && !sets[i].has_vector_types()) return false;
    return true;
  }
  bool has_index_types(unsigned start = 0) const {
    for (size_t i = start; i < sets.size(); i++)
      if (sets[i].size() > 0 && !sets[i].has_indexed_types()) return false;
    return true;
  }

  // Concatenation of the sets from `start` on (reference: src/example.cpp:80-110, 147-228): empty
  // sets are skipped, and with unique_index_types each set's types are shifted past the previous
  // sets'.  Vector types are merged when every non-empty set has them, index types otherwise.
  CoordinateSet merge_coordinates(unsigned start = 0, bool unique_index_types = true) const {
    bool has_vec = has_vector_types(start), has_ind = has_index_types(start);
    if (!has_ind && !has_vec) throw std::invalid_argument("Inconsistent typing schemes in merge_coordinates");
    if (sets.size() <= start) return CoordinateSet();
    if (sets.size() == start + 1) return sets[start].clone();
    if (has_vec) return merge_vector_types(start, unique_index_types);
    std::vector<float3> c;
    std::vector<float> t, r;
    unsigned shift = 0;
    for (size_t s = start; s < sets.size(); s++) {
      const CoordinateSet& cs = sets[s];
      unsigned n = cs.size();
      if (n == 0) continue;
      if (!cs.has_indexed_types())
        throw std::logic_error("Coordinate sets do not have compatible index types for merge.");
      Grid2f cc = cs.coords.cpu();
      Grid1f tt = cs.type_index.cpu(), rr = cs.radii.cpu();
      for (unsigned i = 0; i < n; i++) {
        c.push_back(make_float3(cc(i, 0), cc(i, 1), cc(i, 2)));
        t.push_back(tt(i) + shift);
        r.push_back(rr(i));
      }
      if (unique_index_types) shift += cs.max_type;
    }
    unsigned maxt = 0;
    for (size_t s = start; s < sets.size(); s++)
      maxt = unique_index_types ? maxt + sets[s].max_type : std::max(maxt, sets[s].max_type);
    return CoordinateSet(c, t, r, maxt);
  }

 private:
  // type vectors side by side (or over one another), radii concatenated as they are: per atom, or
  // per type after make_vector_types (src/example.cpp:147-196)
  CoordinateSet merge_vector_types(unsigned start, bool unique_index_types) const {
    unsigned maxt = 0;
    for (size_t i = start; i < sets.size(); i++) {
      maxt = unique_index_types ? maxt + sets[i].max_type : std::max(maxt, sets[i].max_type);
      if (sets[i].size() == 0) continue;
      if (sets[i].max_type != sets[i].type_vector.dimension(1))
        throw std::logic_error("Coordinate set " + itoa(i) + " does not have consistent max_type/vector type sizes");
    }
    std::vector<float3> c;
    std::vector<std::vector<float>> t;
    std::vector<float> r;
    unsigned offset = 0;
    for (size_t s = start; s < sets.size(); s++) {
      const CoordinateSet& cs = sets[s];
      unsigned n = cs.size();
      if (n > 0) {
        Grid2f cc = cs.coords.cpu(), tv = cs.type_vector.cpu();
        unsigned w = (unsigned)tv.dimension(1);
        if (offset + w > maxt) throw std::logic_error("Incompatible vector sizes in merge_coordinates");
        for (unsigned i = 0; i < n; i++) {
          c.push_back(make_float3(cc(i, 0), cc(i, 1), cc(i, 2)));
          std::vector<float> row(maxt, 0.f);
          for (unsigned k = 0; k < w; k++) row[offset + k] = tv(i, k);
          t.push_back(row);
        }
      }
      Grid1f rr = cs.radii.cpu();
      for (unsigned i = 0; i < rr.size(); i++) r.push_back(rr(i));
      if (unique_index_types) offset += cs.max_type;
    }
    CoordinateSet out(c, t, r);
    out.max_type = maxt;
    if (c.empty()) out.type_vector = MGrid2f(0, maxt);
    return out;
  }
};

}  // namespace libmolgrid
#endif
