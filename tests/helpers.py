"""Test helpers: the oracle adapters, re-exported."""
from adapters import MODE_OF, rel_fro, routing, to_oracle_layer  # noqa: F401
