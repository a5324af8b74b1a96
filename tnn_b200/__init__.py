"""tnn_b200 - a Blackwell (B200, sm_100a) native deep-learning framework with the
capabilities of the TNN / tunx reference: layer and model zoo, JSON-config trainer and
inferencer, graph partitioner, pipeline / data / tensor parallel training and the TNNG
checkpoint + archiver wire formats."""
__version__ = "0.1.0"
