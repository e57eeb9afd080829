"""Drop-in for the reference's training-free linear-hash generation modifier
(spotlight/modifiers/linearhashing_generation.py): the same hook, driver and checkpoint format as
``spotlight_generation.Spotlight`` with one ``[1, H, 128, 128]`` projection per layer as the hash
(:224-231). As in the reference (:330-331) layers listed in ``fix_layers`` get no hash module, so
``ft_params()`` holds one tensor per pruned layer."""
from .spotlight_generation import LinearHashingFunction, Spotlight  # noqa: F401


class LinearHashing(Spotlight):
    def __init__(self, model, save_ckp=None, load_ckp=None, config=None):
        super().__init__(model, save_ckp, load_ckp, config, hash_kind="linear")
