"""Spiking ResNet on ImageNet with the classification trainer: a static image is repeated ``--T`` times, the prediction is
the firing rate over time (role of ``model/train_imagenet_example.py`` in the reference).

    python -m spikingjelly_b200.models.train_imagenet_example --T 4 --model spiking_resnet18 --data-path /datasets/ImageNet \\
        --batch-size 64 --lr 0.1 --lr-scheduler cosa --epochs 90
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m spikingjelly_b200.models.train_imagenet_example ...
"""
import torch

from ..activation_based import functional, neuron, surrogate
from . import spiking_resnet, train_classify


class SResNetTrainer(train_classify.Trainer):
    def _repeat(self, args, x: torch.Tensor):
        return x.unsqueeze(0).expand(args.T, *x.shape)            # [N, C, H, W] -> [T, N, C, H, W], no copy

    preprocess_train_sample = preprocess_test_sample = _repeat

    def process_model_output(self, args, y: torch.Tensor):
        return y.mean(0)

    def get_args_parser(self, add_help=True):
        parser = super().get_args_parser(add_help=add_help)
        parser.add_argument("--T", type=int, default=4, help="total time-steps")
        parser.add_argument("--cupy", action="store_true", help="run the neurons on the kernel backend (the reference's flag name)")
        return parser

    def get_tb_logdir_name(self, args):
        return super().get_tb_logdir_name(args) + f"_T{args.T}"

    def load_model(self, args, num_classes):
        builders = [n for n in spiking_resnet.__all__ if n[0].islower()]
        if args.model not in builders:
            raise ValueError(f"args.model should be one of {builders}")
        model = getattr(spiking_resnet, args.model)(pretrained=args.pretrained, spiking_neuron=neuron.IFNode,
                                                    surrogate_function=surrogate.ATan(), detach_reset=True, num_classes=num_classes)
        functional.set_step_mode(model, step_mode="m")
        if args.cupy:
            functional.set_backend(model, "cuda", neuron.IFNode)
        return model


if __name__ == "__main__":
    trainer = SResNetTrainer()
    trainer.main(trainer.get_args_parser().parse_args())
