import sys

from ...internal.experiment import main
from .recipes import RECIPES, config_builder_for

if __name__ == "__main__":
    if len(sys.argv) < 2 or sys.argv[1] not in RECIPES:
        print("usage: python -m olmo_core_b200.scripts.train RECIPE {launch|train|train_single|prep|launch_prep|dry_run} "
              f"RUN_NAME CLUSTER [OVERRIDES...]\nrecipes: {', '.join(sorted(RECIPES))}")
        sys.exit(1)
    recipe = sys.argv.pop(1)
    main(config_builder=config_builder_for(recipe))
