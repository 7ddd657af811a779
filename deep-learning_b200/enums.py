"""Integer codes shared by the C ABI, the Python binding and the parity tests.

The values are those of the reference library's enums so that a caller written
against the reference passes the same numbers
(lib/deep-learning/v1/data/enum/{layer,activation,layer_norm,layer_dropout,
optimizer,loss_fn,model}.hpp).  Only the members the fully-connected training
step supports are listed.
"""


class LAYER:
    FULLY_CONNECTED = 3
    FULLY_CONNECTED_INDEPENDENTLY_RECURRENT = 4
    LSTM = 7
    RESIDUAL = 9


class ACTIVATION:
    ELU = 3
    ISRLU = 10
    LINEAR = 11
    LEAKY_RELU = 14
    RELU = 16
    SELU = 17
    SOFTMAX = 22


class LAYER_NORM:
    NONE = 0
    BATCH_NORMALIZATION = 1
    BATCH_RENORMALIZATION = 2


class LAYER_DROPOUT:
    NONE = 0
    BERNOULLI = 2
    BERNOULLI_INVERTED = 3
    SHAKEDROP = 5
    UOUT = 6


class OPTIMIZER:
    ADABOUND = 1
    ADAM = 2
    ADAMAX = 3
    AMSBOUND = 4
    AMSGRAD = 5
    GD = 6
    NOSADAM = 9


class LOSS_FN:
    CROSS_ENTROPY = 2
    MSE = 10


class MODEL:
    FEEDFORWARD = 3
    RECURRENT = 4
