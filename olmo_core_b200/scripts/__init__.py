"""Command-line utilities: ``python -m olmo_core_b200.scripts.<name>`` (the roles of src/scripts/*.py and src/scripts/train/*)."""
