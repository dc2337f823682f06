"""Sphinx configuration: ``sphinx-build -b html docs docs/_build/html``."""

import os
import sys

sys.path.insert(0, os.path.abspath(".."))

project = "elf-b200"
author = "elf-b200 developers"
release = "0.1.0"

extensions = ["sphinx.ext.autodoc", "sphinx.ext.napoleon", "sphinx.ext.viewcode"]
autodoc_member_order = "bysource"
autodoc_mock_imports = ["elf_b200_C"]
templates_path = ["_templates"]
exclude_patterns = ["_build"]

try:
    import sphinx_rtd_theme  # noqa: F401

    html_theme = "sphinx_rtd_theme"
except ImportError:
    html_theme = "alabaster"
