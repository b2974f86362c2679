#!/usr/bin/env python
"""Training entry point: ``torchrun --nproc_per_node=N train.py --config configs/X.yaml [--flag ...]``
(equivalent to ``python -m kotodama_b200.train``)."""
from kotodama_b200.train import main

if __name__ == "__main__":
    main()
