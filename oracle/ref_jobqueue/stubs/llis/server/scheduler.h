#pragma once
namespace llis { namespace server {
class Server;
class Scheduler {
  public:
    virtual ~Scheduler() {}
    virtual void set_server(Server*) {}
};
} }
