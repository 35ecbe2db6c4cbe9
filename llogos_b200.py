"""Import name of the library in ``daisi-llogos_b200/`` (a folder name Python cannot import
by statement).  ``import llogos_b200 as llogos`` gives the public names; ``python -m llogos_b200``
is the command line.  Sub-packages are reached as attributes (``llogos.engine.Engine``)."""
import importlib as _importlib
import sys as _sys

_pkg = _importlib.import_module("daisi-llogos_b200")
_api = _importlib.import_module("daisi-llogos_b200.api")
_cli = _importlib.import_module("daisi-llogos_b200.cli")
_params = _importlib.import_module("daisi-llogos_b200.sampling.params")
_gen = _importlib.import_module("daisi-llogos_b200.sampling.generate")

LlogosModel = _api.LlogosModel
BenchmarkResult = _api.BenchmarkResult
GenerationParams = _params.GenerationParams
GenerationResult = _gen.GenerationResult
config, weights, parts, cache, engine = _pkg.config, _pkg.weights, _pkg.parts, _pkg.cache, _pkg.engine
load = LlogosModel.load
random_model = LlogosModel.random
__version__ = _pkg.__version__

if __name__ == "__main__":
    _sys.exit(_cli.main())
