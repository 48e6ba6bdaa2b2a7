"""Model zoo matching the reference's examples: MLP, VGG-16/19, ResNet-50/101,
Inception-v4, Transformer encoder-decoder, LSTM."""
from .mlp import mlp
from .vgg import vgg
from .resnet import resnet
from .inception import inception_v4
from .transformer import transformer, TransformerConfig, TransformerModel
from .lstm import lstm
