"""Spiking VGG whose neurons are ``FlexSN`` modules built from a LIF step function written in plain PyTorch (sigmoid
surrogate of slope ``--surrogate-alpha``); the generator compiles the step function into one CUDA kernel per direction
(role of ``model/train_flexsn_inductor_example.py`` in the reference, whose FlexSN backend is Inductor).

    python -m spikingjelly_b200.models.train_flexsn_inductor_example --model spiking_vgg11_bn --data-path /datasets/ImageNet \\
        --batch-size 64 --lr 0.1 --lr-scheduler cosa --epochs 90
"""
import torch

from ..activation_based import functional, surrogate
from ..activation_based.neuron import FlexSN
from . import spiking_vgg, train_classify


class FlexSNTrainer(train_classify.Trainer):
    def _repeat(self, args, x: torch.Tensor):
        return x.unsqueeze(0).expand(args.T, *x.shape)

    preprocess_train_sample = preprocess_test_sample = _repeat

    def process_model_output(self, args, y: torch.Tensor):
        return y.mean(0)

    def get_args_parser(self, add_help=True):
        parser = super().get_args_parser(add_help=add_help)
        parser.add_argument("--T", type=int, default=4, help="total time-steps")
        parser.add_argument("--surrogate-alpha", type=float, default=4.0, help="slope of the sigmoid surrogate gradient")
        parser.add_argument("--flexsn-backend", default="cuda", help="FlexSN backend (the reference's 'inductor' maps to the generated CUDA kernel)")
        return parser

    def get_tb_logdir_name(self, args):
        return super().get_tb_logdir_name(args) + f"_T{args.T}_flexsn_{args.flexsn_backend}_sa{args.surrogate_alpha}"

    def load_model(self, args, num_classes):
        builders = [n for n in spiking_vgg.__all__ if n[0].islower()]
        if args.model not in builders:
            raise ValueError(f"args.model should be one of {builders}")
        sg = surrogate.Sigmoid(alpha=args.surrogate_alpha)

        def lif_core_sg(x: torch.Tensor, v: torch.Tensor):
            h = v + (x - v) / 2.0
            s = sg(h - 1.0)
            return s, h * (1.0 - s)

        def make_flexsn(**kwargs):
            return FlexSN(core=lif_core_sg, num_inputs=1, num_states=1, num_outputs=1, step_mode=kwargs.get("step_mode", "m"),
                          backend=args.flexsn_backend)
        model = getattr(spiking_vgg, args.model)(pretrained=args.pretrained, spiking_neuron=make_flexsn, num_classes=num_classes)
        functional.set_step_mode(model, step_mode="m")
        return model


if __name__ == "__main__":
    trainer = FlexSNTrainer()
    trainer.main(trainer.get_args_parser().parse_args())
