"""Sphinx configuration: ``sphinx-build -b html docs docs/_build``"""
import os
import sys

sys.path.insert(0, os.path.abspath(".."))
project = "returnn-b200"
author = "returnn-b200 developers"
extensions = ["sphinx.ext.autodoc", "sphinx.ext.viewcode"]
master_doc = "index"
exclude_patterns = ["_build"]
html_theme = "alabaster"
autodoc_member_order = "bysource"
