"""Shim package: `utils.runtime` of the reference."""
