"""Model zoo: the headline configurations (VGG-19, ResNet-50, BERT-large) and the other
sequence models of the evaluation set (BERT-base, LSTM language model, Transformer)."""
from .bert import BertConfig, BertForMaskedLM, bert_large, bert_tiny  # noqa: F401
from .resnet import ResNet50, resnet50  # noqa: F401
from .seq import LSTMLanguageModel, TransformerSeq2Seq, bert_base, lstm_lm, transformer_base  # noqa: F401
from .vgg import VGG19, vgg19  # noqa: F401

MODELS = {"vgg19": vgg19, "resnet50": resnet50, "bert_large": bert_large, "bert-large": bert_large,
          "bert_tiny": bert_tiny, "bert_base": bert_base, "lstm": lstm_lm, "transformer": transformer_base}


def get_model(name: str, **kw):
    return MODELS[name.lower()](**kw)
