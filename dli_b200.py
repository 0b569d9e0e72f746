"""Import name of the package whose sources live in ``distributed-llm-inference_b200/``.

The folder's name has a hyphen, so Python cannot import it by that name.  This
module loads the folder as the package ``dli_b200`` and puts it in
``sys.modules`` in its own place: ``import dli_b200`` and
``from dli_b200.engine import LLMEngine`` then work from a checkout without
installation.
"""

import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "distributed-llm-inference_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
