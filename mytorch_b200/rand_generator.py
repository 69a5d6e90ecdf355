"""Seed source for ``uniform_`` / ``normal_`` — behaviour of ``mytorch/rand_generator.py:4-24``:
``manual_seed`` seeds Python's ``random``; every random fill draws one integer in
``[0, 1e9+7]`` from it and uses that as the fill's own seed."""
import random


def manual_seed(meta_seed):
    RandGenerator.instance().reset(meta_seed)


class RandGenerator:
    _instance = None

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self):
        self.reset(0)

    def reset(self, meta_seed):
        random.seed(meta_seed)

    def generate(self):
        return random.randint(0, int(round(1e9 + 7)))
