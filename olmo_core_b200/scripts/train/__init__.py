"""Training recipes: ``python -m olmo_core_b200.scripts.train RECIPE SUBCMD RUN_NAME CLUSTER [overrides]``."""
