from .resnet import ResNet, resnet50, resnet_tiny, to_bf16_channels_last
