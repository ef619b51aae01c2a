"""Glue for experiment scripts: common directories, launch configs, a sub-command CLI and config "cookbook" helpers."""
