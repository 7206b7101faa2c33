"""Model zoo of the headline configurations: VGG-19, ResNet-50, BERT-large."""
from .bert import BertConfig, BertForMaskedLM, bert_large, bert_tiny  # noqa: F401
from .resnet import ResNet50, resnet50  # noqa: F401
from .vgg import VGG19, vgg19  # noqa: F401

MODELS = {"vgg19": vgg19, "resnet50": resnet50, "bert_large": bert_large, "bert-large": bert_large,
          "bert_tiny": bert_tiny}


def get_model(name: str, **kw):
    return MODELS[name.lower()](**kw)
