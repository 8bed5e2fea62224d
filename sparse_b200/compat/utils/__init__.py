"""Shim package: the reference's `utils` module paths over sparse_b200."""
