"""CPU oracle for the quantized-matmul path. Test infrastructure only: the
product package never imports this."""
