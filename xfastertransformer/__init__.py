"""Drop-in import name of the reference package: ``import xfastertransformer`` resolves to
`xfastertransformer_b200` so existing user code keeps working unchanged."""
import sys

import xfastertransformer_b200 as _impl
from xfastertransformer_b200 import *  # noqa: F401,F403
from xfastertransformer_b200 import AutoModel, get_env  # noqa: F401


def __getattr__(name):
    return getattr(_impl, name)
