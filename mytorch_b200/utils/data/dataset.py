"""Dataset base class (``mytorch/utils/data/dataset.py``)."""


class Dataset:
    def __getitem__(self, index):
        raise NotImplementedError()

    def __len__(self):
        raise NotImplementedError()
