"""The synthetic input generators live in the package; tests import them under this name."""
from libmolgrid_b200.synthetic import *  # noqa: F401,F403
