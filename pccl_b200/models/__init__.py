"""models (populated below)."""
