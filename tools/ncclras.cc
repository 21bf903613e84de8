// ncclras: command-line client of the RAS thread. Connects to the RAS client socket of any
// process of the job (default localhost:28028), asks for a status report and prints it.
//   ncclras [-h host] [-p port] [-t seconds] [-f text|json] [-v]
// Reference parity: src/ras/client.cc (options, handshake "CLIENT PROTOCOL", TIMEOUT, STATUS).
#include <netdb.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <string>

static bool sendLine(int fd, const std::string& s) {
  std::string l = s + "\n";
  return send(fd, l.data(), l.size(), MSG_NOSIGNAL) == (ssize_t)l.size();
}
static bool readLine(int fd, std::string* out) {
  out->clear();
  char c;
  while (recv(fd, &c, 1, 0) == 1) {
    if (c == '\n') return true;
    out->push_back(c);
  }
  return !out->empty();
}

int main(int argc, char** argv) {
  const char* host = "localhost";
  const char* port = "28028";
  const char* format = "text";
  int timeout = 5;
  bool verbose = false;
  int opt;
  while ((opt = getopt(argc, argv, "h:p:t:f:v")) != -1) {
    switch (opt) {
      case 'h': host = optarg; break;
      case 'p': port = optarg; break;
      case 't': timeout = atoi(optarg); break;
      case 'f': format = optarg; break;
      case 'v': verbose = true; break;
      default:
        fprintf(stderr, "usage: %s [-h host] [-p port] [-t seconds] [-f text|json] [-v]\n", argv[0]);
        return 2;
    }
  }
  struct addrinfo hints, *res = nullptr;
  memset(&hints, 0, sizeof(hints));
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host, port, &hints, &res) != 0 || !res) { fprintf(stderr, "ncclras: cannot resolve %s:%s\n", host, port); return 1; }
  int fd = -1;
  for (struct addrinfo* a = res; a; a = a->ai_next) {
    fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    if (connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) { fprintf(stderr, "ncclras: no RAS thread answers at %s:%s (is a job running with NCCL_RAS_ENABLE=1?)\n", host, port); return 1; }
  std::string line;
  if (!sendLine(fd, "CLIENT PROTOCOL 2") || !readLine(fd, &line) || line.compare(0, 15, "SERVER PROTOCOL") != 0) { fprintf(stderr, "ncclras: handshake failed\n"); return 1; }
  if (!sendLine(fd, "TIMEOUT " + std::to_string(timeout)) || !readLine(fd, &line) || line != "OK") { fprintf(stderr, "ncclras: TIMEOUT refused\n"); return 1; }
  if (!sendLine(fd, std::string("SET FORMAT ") + format) || !readLine(fd, &line) || line != "OK") { fprintf(stderr, "ncclras: format %s refused\n", format); return 1; }
  if (!sendLine(fd, verbose ? "VERBOSE STATUS" : "STATUS")) return 1;
  char buf[4096];
  ssize_t n;
  while ((n = recv(fd, buf, sizeof(buf), 0)) > 0) fwrite(buf, 1, (size_t)n, stdout);
  close(fd);
  return 0;
}
