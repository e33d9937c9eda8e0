"""Helpers that place the unmodified reference beside this library for comparisons (see make_ref.py)."""
