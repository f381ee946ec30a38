"""Drop-in import name of the reference package: ``import xfastertransformer`` resolves to
`xfastertransformer_b200` so existing user code keeps working unchanged, including
``from xfastertransformer.tools import LlamaConvert`` and the reference's per-family tool modules
(``xfastertransformer.tools.chatglm2_convert`` ...)."""
import importlib
import importlib.abc
import importlib.util
import sys

import xfastertransformer_b200 as _impl
from xfastertransformer_b200 import *  # noqa: F401,F403
from xfastertransformer_b200 import AutoModel, get_env  # noqa: F401
from xfastertransformer_b200 import tools as _tools

sys.modules[__name__ + ".tools"] = _tools
tools = _tools


class _ToolModules(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """``import xfastertransformer.tools.<reference module name>`` -> the module of this package with those classes."""

    prefix = __name__ + ".tools."

    def find_spec(self, fullname, path=None, target=None):
        if fullname.startswith(self.prefix) and fullname[len(self.prefix):] in _tools.REFERENCE_MODULES:
            return importlib.util.spec_from_loader(fullname, self)
        return None

    def create_module(self, spec):
        return importlib.import_module("xfastertransformer_b200.tools." +
                                       _tools.REFERENCE_MODULES[spec.name[len(self.prefix):]])

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _ToolModules())


def __getattr__(name):
    return getattr(_impl, name)
