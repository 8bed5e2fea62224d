"""Shim package: the reference's `scripts` launchers over sparse_b200."""
