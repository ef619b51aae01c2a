"""Launching jobs: on the local node with ``torchrun`` (:mod:`.local`) or on a Beaker cluster (:mod:`.beaker`)."""
