"""VGG-19 (16 conv + 3 FC, 143.7 M parameters), the model of the reference's
headline launch line (``--model vgg19``, README.md:45 of mark14wu/hipress).
Parameter names and sizes follow the MXNet gluon numbering of the reference's
SeCoPa sample input (src/SeCoPa/input.txt): conv0..conv15, dense0..dense2."""
import torch
import torch.nn as nn

CFG19 = [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M",
         512, 512, 512, 512, "M"]


class VGG19(nn.Module):
    def __init__(self, num_classes: int = 1000, dropout: float = 0.5):
        super().__init__()
        layers, cin = [], 3
        for v in CFG19:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(cin, v, 3, padding=1), nn.ReLU(inplace=True)]
                cin = v
        self.features = nn.Sequential(*layers)
        self.classifier = nn.Sequential(
            nn.Linear(512 * 7 * 7, 4096), nn.ReLU(inplace=True), nn.Dropout(dropout),
            nn.Linear(4096, 4096), nn.ReLU(inplace=True), nn.Dropout(dropout),
            nn.Linear(4096, num_classes))
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
                nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        x = self.features(x)
        return self.classifier(torch.flatten(x, 1))

    def gluon_named_parameters(self):
        """(name, parameter) with the reference's gradient names, e.g.
        ``vgg0_conv0_weight`` ... ``vgg0_dense2_bias``."""
        ci = di = 0
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                yield f"vgg0_conv{ci}_weight", m.weight
                yield f"vgg0_conv{ci}_bias", m.bias
                ci += 1
            elif isinstance(m, nn.Linear):
                yield f"vgg0_dense{di}_weight", m.weight
                yield f"vgg0_dense{di}_bias", m.bias
                di += 1


def vgg19(**kw):
    return VGG19(**kw)
