// Link-time stand-ins for the stb_image entry points that the reference's image-folder loaders
// declare. The stb headers are fetched from the network by the reference's CMake project and are
// not available offline; the synthetic-data benchmark never decodes an image file, so these only
// have to exist. Every one reports failure.
extern "C" {
unsigned char* stbi_load(const char*, int*, int*, int*, int) { return nullptr; }
void stbi_image_free(void*) {}
unsigned char* stbi_load_from_memory(unsigned char const*, int, int*, int*, int*, int) { return nullptr; }
unsigned char* stbir_resize_uint8_linear(const unsigned char*, int, int, int, unsigned char*, int, int, int, int) {
  return nullptr;
}
const char* stbi_failure_reason(void) { return "stb_image is not available in this build"; }
}
