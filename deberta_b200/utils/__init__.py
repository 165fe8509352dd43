"""Small shared helpers (typing coercion, mappings, serialisation, atomic IO, logging)."""
