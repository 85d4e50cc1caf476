"""Small dependency-free helpers."""
