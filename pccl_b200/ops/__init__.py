"""ops (populated below)."""
