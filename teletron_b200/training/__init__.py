"""Training runtime: flags, initialisation, the step loop, optimizer, checkpoints, logging."""

from .args import get_args, parse_args  # noqa: F401
from .logging import print_rank_0  # noqa: F401
from .pretrain import (  # noqa: F401
    average_losses_across_data_parallel_group,
    build_train_valid_test_data_iterators,
    get_timers,
    initialize,
    pretrain,
    setup_model_and_optimizer,
    train,
    train_step,
)
