// Stand-in for boost::lexical_cast, used by the reference only to format numbers into strings.
#pragma once
#include <sstream>
#include <string>
namespace boost {
template <class Target, class Source>
Target lexical_cast(const Source& s) {
  std::ostringstream os;
  os << s;
  return Target(os.str());
}
}  // namespace boost
