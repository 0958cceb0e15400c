} // namespace ref_host
extern "C" unsigned ref_index(unsigned input_in_tile, unsigned output_in_tile) {
  return ref_host::Index(input_in_tile, output_in_tile);
}
// FP32 value of one weight exactly as the reference's scalar decoder returns it.
extern "C" float ref_weight(const unsigned char *data, int rows, int cols, int format, int input, int output) {
  DeviceMatrix m;
  m.data = data;
  m.rows = rows;
  m.cols = cols;
  m.format = format;
  return ref_host::Weight(m, input, output);
}
extern "C" void ref_decode_matrix(const unsigned char *data, int rows, int cols, int format, float *out) {
  DeviceMatrix m;
  m.data = data;
  m.rows = rows;
  m.cols = cols;
  m.format = format;
  for (int i = 0; i < cols; ++i)
    for (int o = 0; o < rows; ++o)
      out[static_cast<std::size_t>(i) * rows + o] = ref_host::Weight(m, i, o);
}
