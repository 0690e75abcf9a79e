"""B200-native SGEMM backend: generator (CUDA source + cubin + TOML), runner (C ABI over the CUDA driver),
tuner.  The sub-packages keep the reference project's module paths (``generator.generator``,
``tuner.sgemm_tuner``), which it uses with its checkout root on ``PYTHONPATH``; importing this package
puts its own directory on ``sys.path`` so the same imports resolve here."""
import sys as _sys
from pathlib import Path as _Path

PACKAGE_DIR = _Path(__file__).resolve().parent
if str(PACKAGE_DIR) not in _sys.path:
    _sys.path.insert(0, str(PACKAGE_DIR))
