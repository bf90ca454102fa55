"""Plug-in modules for the reference project's benchmark harness.

The harness discovers candidates by scanning the source text of the modules in
its `bench/candidates/` folder for literal `NAME = "..."` and `VARIANT = "..."`
lines (bench/bench/candidates/__init__.py:22-46).  Copy or symlink the modules
of this folder there; nothing else of the harness changes."""
