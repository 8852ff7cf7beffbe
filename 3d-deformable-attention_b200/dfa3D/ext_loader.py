"""``load_ext`` with the reference's contract (DFA3D/dfa3D/ext_loader.py:25-29): import the named
extension of this package and assert that it has the requested functions."""
import importlib


def load_ext(name, funcs):
    ext = importlib.import_module('dfa3D.' + name)
    for fun in funcs:
        assert hasattr(ext, fun), f'{fun} miss in module {name}'
    return ext
