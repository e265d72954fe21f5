"""`repop.backend`: per-device raw entry points (seeding, raw GEMMs for the streaming vocabulary head)."""
