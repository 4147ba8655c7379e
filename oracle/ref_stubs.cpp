/* TEST INFRASTRUCTURE ONLY.
 * Link-time stand-ins for two reference functions that the Example/CoordinateSet
 * overloads of GridMaker reference but that the oracle never calls (their
 * definitions live in translation units that need OpenBabel).  Reaching one aborts.
 */
#include <cstdlib>

#include "libmolgrid/coordinateset.h"
#include "libmolgrid/example.h"

namespace libmolgrid {
float3 CoordinateSet::center() const { std::abort(); }
CoordinateSet Example::merge_coordinates(unsigned, bool) const { std::abort(); }
}  // namespace libmolgrid
