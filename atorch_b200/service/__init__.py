"""gRPC planes of the data path: coworker processing / batch serving and the data-info directory."""
