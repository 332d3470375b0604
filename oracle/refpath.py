"""Where the reference checkout (dnvtmf/Fast-SP-GS) lives.  Test infrastructure only."""
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root(explicit=None):
    """The directory that holds ``fast_2d_gs/``: ``explicit`` when given, else ``$FSGS_REFERENCE_ROOT``, else a
    directory called ``reference`` next to this repository.  Returns None when none of them exists."""
    candidates = [explicit, os.environ.get("FSGS_REFERENCE_ROOT"),
                  os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in candidates:
        if c and os.path.isdir(os.path.join(c, "fast_2d_gs", "_C")):
            return os.path.abspath(c)
    return None
