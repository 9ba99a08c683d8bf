from .optim import Q_Adafactor, Q_AdamW, Q_AGD, Q_CAME
