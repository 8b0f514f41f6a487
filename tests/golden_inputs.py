"""Loads tests/golden/make_ref_fixtures.py as a module so tests regenerate the fixture inputs with the
exact code that produced the fixture."""
import importlib.util
import os

_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_ref_fixtures.py")
_spec = importlib.util.spec_from_file_location("make_ref_fixtures", _path)
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)
