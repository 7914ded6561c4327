from .registry import DATASETS, Registry, build_dataset, build_module  # noqa: F401
from .fake_dataset import FakeDataset  # noqa: F401
from .koala_dataset import KoalaDataset  # noqa: F401
from .loader import build_pretraining_data_loader  # noqa: F401
