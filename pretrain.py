"""``torchrun … pretrain.py --flags``: the training entry point (see archscale_b200/train/pretrain.py)."""
from archscale_b200.train.pretrain import main

if __name__ == "__main__":
    main()
