"""Serialization registry (filled in by opake_b200.base._serialization_impl)."""
