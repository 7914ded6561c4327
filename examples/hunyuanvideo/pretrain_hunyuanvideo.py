"""HunyuanVideo pre-training entry point (counterpart of the reference's
``examples/hunyuanvideo/pretrain_hunyuanvideo.py:48-171``): provides the extra flags, the model,
the dataset and the forward step to :func:`teletron_b200.training.pretrain`."""

import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))

import torch  # noqa: E402

from teletron_b200.data import build_dataset  # noqa: E402
from teletron_b200.encoder_service import producer_process  # noqa: E402
from teletron_b200.models.hunyuanvideo import (FlowConfig, HunyuanPipeline, hunyuan_13b, sanity_config,  # noqa: E402
                                               tiny_config)
from teletron_b200.training import (average_losses_across_data_parallel_group, get_args, get_timers,  # noqa: E402
                                    pretrain)
from teletron_b200.training.batch import get_batch_on_this_tp_cp_rank  # noqa: E402
from teletron_b200.training.logging import model_flops_per_sample, print_rank_0  # noqa: E402


def extra_args_provider(parser):
    g = parser.add_argument_group("hunyuanvideo")
    g.add_argument("--text-len", type=int, default=256, help="text tokens per sample (FakeDataset)")
    g.add_argument("--with-vae", action="store_true", help="encode pixels on the DiT ranks (no encoder service)")
    return parser


def build_config(args):
    make = {"13b": hunyuan_13b, "sanity": sanity_config, "tiny": tiny_config}[args.model_size]
    kw = dict(recompute_granularity=args.recompute_granularity, recompute_method=args.recompute_method,
              recompute_num_layers=None, init_method_std=args.init_method_std, seed=args.seed,
              apply_text_mask=args.apply_text_mask, recompute_save_attention=args.recompute_save_attention,
              sequence_parallel=bool(args.sequence_parallel), sequence_pad_multiple=args.sequence_pad_multiple)
    if args.model_size != "tiny":
        kw["in_channels"] = 33 if args.model_type == "i2v" else 16
    cfg = make(**kw).apply_env_overrides()
    if args.dit_num_layers is not None:
        cfg.num_layers = args.dit_num_layers
    if args.dit_num_single_layers is not None:
        cfg.num_single_layers = args.dit_num_single_layers
    return cfg


def model_provider():
    args = get_args()
    cfg = build_config(args)
    flow = FlowConfig(shift=args.flow_shift, weighting_scheme=args.flow_weighting_scheme,
                      logit_mean=args.flow_logit_mean, logit_std=args.flow_logit_std,
                      mode_scale=args.flow_mode_scale, sanity_check=args.sanity_check,
                      model_type=args.model_type if args.model_size != "tiny" else "t2v")
    vae = None
    if args.with_vae and not args.distributed_vae:
        from teletron_b200.models.vae import AutoencoderKLHunyuanVideo
        vae = AutoencoderKLHunyuanVideo().to(args.device, args.params_dtype)
        vae.enable_tiling(not args.vae_tiling is False)
    print_rank_0(f"building HunyuanVideo MMDiT: {cfg.num_layers} dual + {cfg.num_single_layers} single blocks, "
                 f"hidden {cfg.hidden_size}")
    pipe = HunyuanPipeline(cfg, flow, vae=vae, device=args.device, dtype=args.params_dtype)
    pipe._placed = True
    W, H = args.video_resolution
    f = (args.num_frames - 1) // 4 + 1
    tokens = f * (H // 16) * (W // 16)
    args.tokens_per_sample = tokens + args.text_len
    args.flops_per_sample = model_flops_per_sample(cfg.num_parameters(), tokens, args.text_len,
                                                   cfg.num_attention_heads, cfg.attention_head_dim,
                                                   cfg.num_layers + cfg.num_single_layers,
                                                   False)        # useful FLOPs: what an MFU is quoted on
    return pipe


def loss_func(output_tensor):
    loss = output_tensor[0].mean()
    averaged = average_losses_across_data_parallel_group([loss])
    return loss, {"loss": averaged[0]}


def forward_step(data_iterator, model):
    args = get_args()
    timers = get_timers()
    timers("batch-generator", log_level=2).start()
    pipe = model.module
    encode = pipe.forward_vae if pipe.vae is not None else None
    batch = get_batch_on_this_tp_cp_rank(data_iterator, args.device, consumer=getattr(args, "encoder_consumer", None),
                                         encode_fn=encode)
    timers("batch-generator").stop()
    return model(batch), loss_func


def train_valid_test_datasets_provider(train_val_test_num_samples):
    args = get_args()
    tiny = args.model_size == "tiny"
    kw = dict(num_frames=args.num_frames, video_resolution=args.video_resolution, koala_opt=args.koala_opt,
              text_len=args.text_len, text_dim=64 if tiny else 4096, pooled_dim=32 if tiny else 768,
              with_pixels=bool(args.with_vae or args.distributed_vae))
    ds = build_dataset(args.dataset_type, **kw)
    valid = None
    if args.eval_iters > 0 and args.dataset_type == "FakeDataset":
        valid = build_dataset(args.dataset_type, seed=1, **kw)        # held-out synthetic items
    return ds, valid, None


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             producer_process=producer_process, extra_args_provider=extra_args_provider)
