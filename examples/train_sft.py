"""DP supervised fine-tuning: the ``sft`` command of ``python -m opake_b200.cli`` (presets, model / data / privacy / sharding options:
``python examples/train_sft.py --help``; quick check on a CPU: ``python examples/train_sft.py --preset smoke --cpu --stop-at-step 3``)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opake_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    main(["sft", *sys.argv[1:]])
