"""One-off dataset preparation helpers (API of src/olmo_core/data/misc)."""
