"""pytest plugin (``-p reference_alias_plugin``) that makes ``import torchtitan[.x.y]`` resolve to
``torchtitan_b200[.x.y]``: the reference's own unit tests then exercise this package. Used by
``test_reference_unit_tests.py`` in a child process; never loaded by this repository's own test session."""

import importlib
import importlib.abc
import importlib.util
import sys
import types
import unittest

_SRC, _DST = "torchtitan", "torchtitan_b200"


class _Alias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name != _SRC and not name.startswith(_SRC + "."):
            return None
        real = _DST + name[len(_SRC):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(name, self, is_package=True)

    def create_module(self, spec):
        mod = importlib.import_module(_DST + spec.name[len(_SRC):])
        sys.modules[spec.name] = mod               # the same module object under both names: patches reach the code
        return mod

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _Alias())

if importlib.util.find_spec("expecttest") is None:      # only its TestCase base class is used
    _m = types.ModuleType("expecttest")

    class _TestCase(unittest.TestCase):
        def assertExpectedInline(self, actual, expect, skip=0):
            self.assertEqual(str(actual).strip(), str(expect).strip())

    _m.TestCase = _TestCase
    sys.modules["expecttest"] = _m
