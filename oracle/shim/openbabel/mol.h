// Forward declarations only: the oracle never builds a CoordinateSet from an OBMol.
#pragma once
namespace OpenBabel { class OBMol; class OBAtom; }
